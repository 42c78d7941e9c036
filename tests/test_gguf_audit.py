"""The loader's audit of a checkpoint, on a machine without a GPU: container, family spec and every decoder tensor
(presence, shape, block format, nothing of another layer kind), as the reference checks them before it builds a model
(src/gguf.rs:2155-2220, src/gguf_model.rs:3388-3776).  Valid seed checkpoints of the five families must pass with the
right summary; files broken in one place each must be refused with a message that names the place."""
import importlib
import struct

import numpy as np
import pytest


@pytest.fixture(scope="module")
def pk(mk):
    return dict(eng=importlib.import_module("macllm_infer_b200.engine"), seed=importlib.import_module("macllm_infer_b200.seed_gguf"),
                capi=importlib.import_module("macllm_infer_b200._capi"))


FAMILIES = {
    "llama": dict(name="tinyllama-1.1b", layers=2, vocab=512, hidden=256, ffn=512),
    "smollm3": dict(name="smollm3-3b", layers=4, vocab=512, hidden=256, ffn=512),
    "qwen3": dict(name="qwen3-8b", layers=2, vocab=512, hidden=256, ffn=512),
    "gemma2": dict(name="gemma2-9b", layers=2, vocab=512, hidden=256, ffn=512, window=24),
    "qwen3moe": dict(name="qwen3-30b-a3b", layers=2, vocab=512, hidden=256, experts=8),
}


def spec_of(pk, fam):
    kw = dict(FAMILIES[fam])
    return pk["seed"].scaled(kw.pop("name"), **kw)


def write_structure(pk, path, metas, plan, magic=None, version=3, truncate=0):
    """A GGUF file with the given metadata records and tensor descriptors and zero-filled data."""
    seed = pk["seed"]
    sizes = {16: 66}  # IQ2_XXS, a format neither the reference's loader nor this path reads
    def nbytes(dims, qtype):
        return int(np.prod(dims)) // 256 * sizes[qtype] if qtype in sizes else seed._tensor_bytes(dims, qtype)
    head = struct.pack("<IIQQ", seed.GGUF_MAGIC if magic is None else magic, version, len(plan), len(metas)) + b"".join(metas)
    offset = 0
    for name, dims, qtype, _ in plan:
        head += seed._s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in reversed(dims)) + struct.pack("<IQ", qtype, offset)
        offset += (nbytes(dims, qtype) + seed.ALIGN - 1) // seed.ALIGN * seed.ALIGN
    head += b"\0" * ((-len(head)) % seed.ALIGN)
    with open(path, "wb") as f:
        f.write(head + b"\0" * max(0, offset - truncate))
    return path


@pytest.mark.parametrize("fam", list(FAMILIES))
def test_seed_checkpoints_pass_with_the_right_summary(pk, tmp_path, fam):
    seed = pk["seed"]
    spec = spec_of(pk, fam)
    path = seed.write_seed_gguf(tmp_path / f"{fam}.gguf", spec, seed=0)
    s = pk["eng"].Model.inspect_gguf(path)
    assert s["architecture"] == spec.arch
    assert (s["n_layers"], s["hidden_size"], s["q_heads"], s["kv_heads"], s["head_dim"]) == (spec.layers, spec.hidden, spec.q_heads, spec.kv_heads, spec.head_dim)
    assert s["vocab_size"] == spec.vocab and s["max_context"] == spec.context and s["tied_embeddings"] == int(spec.tied)
    assert (s["experts"], s["experts_used"], s["expert_ffn_size"]) == (spec.experts, spec.experts_used, spec.expert_ffn)
    plan = seed.tensor_plan(spec)
    assert s["tensors_in_file"] == len(plan) == s["matrices"] + s["vectors"]
    # the seed module counts every 2-D tensor; the audit files the F32 router under the vectors
    assert s["matrix_bytes"] == seed.weight_bytes(spec)["total"] - spec.experts * spec.hidden * 4 * spec.layers
    assert s["sliding_layers"] == (spec.layers // 2 if fam == "gemma2" else 0)
    assert s["nope_layers"] == (spec.layers // 4 if fam == "smollm3" else 0)
    assert s["qk_norm"] == int(fam in ("qwen3", "qwen3moe"))


def broken(pk, tmp_path, fam, edit, **kw):
    seed = pk["seed"]
    spec = spec_of(pk, fam)
    metas, plan = seed._meta(spec), list(seed.tensor_plan(spec))
    metas, plan = edit(spec, metas, plan) or (metas, plan)
    return write_structure(pk, tmp_path / "broken.gguf", metas, plan, **kw)


def refused(pk, path, fragment):
    with pytest.raises(pk["capi"].MkError) as e:
        pk["eng"].Model.inspect_gguf(path)
    assert fragment in str(e.value), str(e.value)


def test_structural_copy_of_a_valid_file_passes(pk, tmp_path):
    path = broken(pk, tmp_path, "qwen3", lambda spec, m, p: None)
    assert pk["eng"].Model.inspect_gguf(path)["n_layers"] == 2


def test_missing_tensor_is_named(pk, tmp_path):
    path = broken(pk, tmp_path, "llama", lambda s, m, p: (m, [t for t in p if t[0] != "blk.1.ffn_up.weight"]))
    refused(pk, path, "required GGUF tensor `blk.1.ffn_up.weight` is missing")


def test_wrong_shape_reports_found_and_expected(pk, tmp_path):
    def edit(spec, m, p):
        return m, [(n, (d[0], d[1] * 2) if n == "blk.0.attn_k.weight" else d, q, s) for n, d, q, s in p]
    refused(pk, broken(pk, tmp_path, "qwen3", edit), "GGUF tensor `blk.0.attn_k.weight` has shape [1024, 512], expected [1024, 256]")


def test_bias_tensors_are_refused_not_ignored(pk, tmp_path):
    f32 = pk["capi"].TYPE_F32
    path = broken(pk, tmp_path, "qwen3", lambda spec, m, p: (m, p + [("blk.0.attn_q.bias", (spec.q_heads * spec.head_dim,), f32, 0.0)]))
    refused(pk, path, "carries a bias tensor")


def test_dense_layer_with_expert_tensors_and_moe_layer_with_dense_tensors(pk, tmp_path):
    f32 = pk["capi"].TYPE_F32
    refused(pk, broken(pk, tmp_path, "llama", lambda spec, m, p: (m, p + [("blk.0.ffn_gate_inp.weight", (8, spec.hidden), f32, 0.0)])),
            "dense layer 0 contains incompatible sparse-MoE tensor `ffn_gate_inp.weight`")
    q4 = pk["capi"].TYPE_Q4_K
    refused(pk, broken(pk, tmp_path, "qwen3moe", lambda spec, m, p: (m, p + [("blk.1.ffn_up.weight", (512, spec.hidden), q4, 0.0)])),
            "sparse-MoE layer 1 contains unsupported dense tensor `ffn_up.weight`")


def test_tensor_of_another_sequence_mixer(pk, tmp_path):
    f32 = pk["capi"].TYPE_F32
    path = broken(pk, tmp_path, "llama", lambda spec, m, p: (m, p + [("blk.0.ssm_a", (4,), f32, 0.0)]))
    refused(pk, path, "attention layer 0 contains a tensor of another sequence mixer: `ssm_a`")


def test_block_formats(pk, tmp_path):
    def retype(name, qtype):
        return lambda spec, m, p: (m, [(n, d, qtype if n == name else q, s) for n, d, q, s in p])
    refused(pk, broken(pk, tmp_path, "llama", retype("blk.0.ffn_down.weight", 16)),
            "unsupported GGML tensor type 16; this runtime currently supports F32 (0), F16 (1), Q4_0 (2)")
    refused(pk, broken(pk, tmp_path, "llama", retype("blk.0.attn_norm.weight", pk["capi"].TYPE_F16)), "`blk.0.attn_norm.weight` must be F32")


def test_container_errors(pk, tmp_path):
    same = lambda spec, m, p: None
    refused(pk, broken(pk, tmp_path, "llama", same, magic=0x12345678), "is not a GGUF file")
    refused(pk, broken(pk, tmp_path, "llama", same, version=1), "unsupported GGUF version 1")
    refused(pk, broken(pk, tmp_path, "llama", same, truncate=4096), "extends past the end of the file")
    refused(pk, tmp_path / "nothing-here.gguf", "cannot open GGUF file")


def test_metadata_errors(pk, tmp_path):
    seed = pk["seed"]
    def drop(key):
        return lambda spec, m, p: ([r for r in m if not r.startswith(seed._s(key))], p)
    refused(pk, broken(pk, tmp_path, "llama", drop("llama.block_count")), "GGUF metadata key `llama.block_count` is missing")
    def other_arch(spec, m, p):
        return [seed._kv("general.architecture", seed.T_STR, seed._s("mamba2")) if r.startswith(seed._s("general.architecture")) else r for r in m], p
    refused(pk, broken(pk, tmp_path, "llama", other_arch), "architecture `mamba2` is not supported on this path")
    refused(pk, broken(pk, tmp_path, "llama", drop("general.quantization_version")), "quantized GGUF tensors require general.quantization_version")
    def old_quant(spec, m, p):
        key = "general.quantization_version"
        return [seed._kv(key, seed.T_U32, struct.pack("<I", 1)) if r.startswith(seed._s(key)) else r for r in m], p
    refused(pk, broken(pk, tmp_path, "llama", old_quant), "unsupported GGUF quantization version 1; expected version 2")
    def heads(spec, m, p):
        key = "qwen3.attention.head_count_kv"
        return [seed._kv(key, seed.T_U32, struct.pack("<I", 3)) if r.startswith(seed._s(key)) else r for r in m], p
    refused(pk, broken(pk, tmp_path, "qwen3", heads), "query heads must be a multiple of KV heads")


def test_rope_frequency_factors_are_read_for_llama_only(pk, tmp_path):
    """src/gguf_model.rs:1855,2015-2033 (Llama reads head_dim / 2 finite positive factors) and :1302,2138 (the other
    profiles refuse the tensor)."""
    seed, f32 = pk["seed"], pk["capi"].TYPE_F32
    def with_factors(n):
        return lambda spec, m, p: (m, p + [("rope_freqs.weight", (n,), f32, 0.0)])
    spec = spec_of(pk, "llama")
    # zero-filled payload: the right length but not positive
    refused(pk, broken(pk, tmp_path, "llama", with_factors(spec.head_dim // 2)), "factors must be finite and positive")
    refused(pk, broken(pk, tmp_path, "llama", with_factors(3)), f"`rope_freqs.weight` has 3 factors, expected {spec.head_dim // 2} for head dimension {spec.head_dim}")
    refused(pk, broken(pk, tmp_path, "qwen3", with_factors(64)), "GGUF qwen3 rope frequency factors are not supported yet")
    refused(pk, broken(pk, tmp_path, "gemma2", with_factors(128)), "GGUF Gemma 2 RoPE frequency-factor tensors are not supported")
    good = seed.scaled("tinyllama-1.1b", layers=2, vocab=512, hidden=256, ffn=512)
    good.extra = dict(good.extra, rope_factors=np.linspace(1.0, 8.0, good.head_dim // 2))
    s = pk["eng"].Model.inspect_gguf(seed.write_seed_gguf(tmp_path / "factors.gguf", good, seed=0))
    assert s["tensors_in_file"] == s["matrices"] + s["vectors"] + 1


def test_shard_family_is_one_checkpoint(pk, tmp_path):
    """src/gguf.rs:576-660: a family `<prefix>-00001-of-0000n.gguf` opened through its first member holds the tensors of
    all members and the metadata of the first."""
    seed = pk["seed"]
    spec = spec_of(pk, "qwen3")
    whole = pk["eng"].Model.inspect_gguf(seed.write_seed_gguf(tmp_path / "whole.gguf", spec, seed=0))
    first = seed.write_seed_gguf_shards(tmp_path / "fam", "model", spec, 3, seed=0)
    assert first.name == "model-00001-of-00003.gguf"
    assert pk["eng"].Model.inspect_gguf(first) == whole


def test_shard_family_rules(pk, tmp_path):
    seed = pk["seed"]
    spec = spec_of(pk, "llama")
    plan, n = seed.tensor_plan(spec), len(seed.tensor_plan(spec))
    half = n // 2
    def family(d, first_metas=None, second_metas=None, first_plan=None, second_plan=None, names=("m-00001-of-00002.gguf", "m-00002-of-00002.gguf")):
        d.mkdir()
        arch = [seed._kv("general.architecture", seed.T_STR, seed._s(spec.arch))]
        write_structure(pk, d / names[0], first_metas if first_metas is not None else seed._meta(spec) + seed.split_metas(0, 2, n),
                        plan[:half] if first_plan is None else first_plan)
        if names[1] is not None:
            write_structure(pk, d / names[1], second_metas if second_metas is not None else arch + seed.split_metas(1, 2, n),
                            plan[half:] if second_plan is None else second_plan)
        return d / names[0]
    arch = [seed._kv("general.architecture", seed.T_STR, seed._s(spec.arch))]
    assert pk["eng"].Model.inspect_gguf(family(tmp_path / "ok"))["tensors_in_file"] == n
    refused(pk, family(tmp_path / "gone", names=("m-00001-of-00002.gguf", None)), "failed to load GGUF shard 2 of 2")
    refused(pk, family(tmp_path / "no", second_metas=arch + seed.split_metas(0, 2, n)), "declares split.no=0, expected 1")
    refused(pk, family(tmp_path / "count", second_metas=arch + seed.split_metas(1, 3, n)), "declares split.count=3, expected 2")
    refused(pk, family(tmp_path / "total", second_metas=arch + seed.split_metas(1, 2, n + 1)), f"declares split.tensors.count={n + 1}, expected {n}")
    refused(pk, family(tmp_path / "nosplit", second_metas=arch), "is missing required split metadata")
    refused(pk, family(tmp_path / "short", second_plan=plan[half:-1]), f"declares {n} tensors, but {n - 1} unique tensors were loaded")
    refused(pk, family(tmp_path / "twice", second_plan=plan[half - 1:-1]), "appears more than once")
    extra = arch + [seed._kv("llama.block_count", seed.T_U32, struct.pack("<I", 99))] + seed.split_metas(1, 2, n)
    refused(pk, family(tmp_path / "conflict", second_metas=extra), "has conflicting metadata `llama.block_count`")
    added = arch + [seed._kv("general.note", seed.T_STR, seed._s("x"))] + seed.split_metas(1, 2, n)
    refused(pk, family(tmp_path / "added", second_metas=added), "contains metadata `general.note` absent from the first shard")
    # the family must be entered through its first member, and names and metadata must tell the same story
    ok_second = tmp_path / "ok" / "m-00002-of-00002.gguf"
    refused(pk, ok_second, "has split.no=1; load the first shard instead")
    refused(pk, family(tmp_path / "name", names=("plain.gguf", "m-00002-of-00002.gguf")), "does not match split.no=0 and split.count=2")
    refused(pk, family(tmp_path / "meta", first_metas=seed._meta(spec), first_plan=plan, names=("m-00001-of-00002.gguf", None)),
            "declares an active shard family, but its metadata does not")


def test_oracle_reads_a_shard_family_like_the_single_file(pk, tmp_path):
    """The oracle's reader follows the same family rule, so sharded checkpoints can be compared with the product."""
    from oracle import decoder
    seed = pk["seed"]
    spec = spec_of(pk, "qwen3")
    whole = decoder.Gguf(seed.write_seed_gguf(tmp_path / "whole.gguf", spec, seed=0))
    family = decoder.Gguf(seed.write_seed_gguf_shards(tmp_path / "fam", "model", spec, 3, seed=0))
    assert len(family.members) == 3 and set(family.tensors) == set(whole.tensors)
    for name in whole.tensors:
        a, b = whole.raw(name), family.raw(name)
        assert a[1:] == b[1:] and np.array_equal(a[0], b[0]), name


# ---- the container parser's own rules (parse_gguf, src/gguf.rs:2069-2240; its tests at src/gguf.rs:3748-3862) ---------------

def raw_gguf(seed, metas=(), tensors=(), version=3, counts=None, align=32, pad_data=True):
    """A bare GGUF file: `metas` are encoded records, `tensors` are (name, file-order dims, type tag, payload bytes, offset or
    None for the canonical one)."""
    n_t, n_kv = counts if counts is not None else (len(tensors), len(metas))
    head = struct.pack("<IIQQ", seed.GGUF_MAGIC, version, n_t, n_kv) + b"".join(metas)
    offset, data = 0, b""
    for name, dims, tag, payload, off in tensors:
        head += seed._s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", tag, offset if off is None else off)
        padded = payload + b"\0" * ((-len(payload)) % align)
        data += padded
        offset += len(padded)
    if tensors:
        head += b"\0" * ((-len(head)) % align)
    return head + (data if pad_data else b"")


def refused_bytes(pk, tmp_path, blob, fragment):
    path = tmp_path / "raw.gguf"
    path.write_bytes(blob)
    with pytest.raises(pk["capi"].MkError) as e:
        pk["eng"].Model.inspect_gguf(path)
    assert fragment in str(e.value), str(e.value)


def f32s(*values):
    return struct.pack(f"<{len(values)}f", *values)


def test_rejects_bad_magic_version_and_header_counts(pk, tmp_path):
    """src/gguf.rs:3748-3767."""
    seed = pk["seed"]
    valid = raw_gguf(seed)
    refused_bytes(pk, tmp_path, b"X" + valid[1:], "bad GGUF magic")
    refused_bytes(pk, tmp_path, valid[:4] + struct.pack("<I", 2) + valid[8:], "unsupported GGUF version 2; expected version 3")
    refused_bytes(pk, tmp_path, valid[:4] + struct.pack(">I", 3) + valid[8:], "big-endian GGUF v3 is not supported")
    refused_bytes(pk, tmp_path, valid[:8] + struct.pack("<Q", 2 ** 64 - 1) + valid[16:], "GGUF tensor count 18446744073709551615 exceeds limit 1048576")
    refused_bytes(pk, tmp_path, raw_gguf(seed, counts=(1000, 1000)), "declared tensor/metadata counts need at least 37000 bytes, but only 0 remain")
    refused_bytes(pk, tmp_path, valid[:10], "unexpected end of GGUF file at byte 8 while reading 8 bytes")


def test_rejects_duplicate_metadata_and_tensor_names(pk, tmp_path):
    """src/gguf.rs:3769-3786."""
    seed = pk["seed"]
    kv = lambda v: seed._kv("same", seed.T_U32, struct.pack("<I", v))
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=[kv(1), kv(2)]), "duplicate GGUF metadata key 'same'")
    t = ("same", (1,), 0, f32s(1.0), None)
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[t, t]), "duplicate GGUF tensor name 'same'")


def test_rejects_invalid_bool_unknown_type_and_nested_array(pk, tmp_path):
    """src/gguf.rs:3788-3807."""
    seed = pk["seed"]
    T_BOOL, T_ARRAY, T_U8 = 7, 9, 0
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=[seed._kv("bool", T_BOOL, b"\x02")]), "invalid GGUF boolean byte 2; expected 0 or 1")
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=[seed._kv("value", 99, struct.pack("<I", 1))]), "unknown GGUF metadata value type 99")
    nested = struct.pack("<IQ", T_ARRAY, 1) + struct.pack("<IQ", T_U8, 0)
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=[seed._kv("nested", T_ARRAY, nested)]), "nested GGUF metadata arrays are not supported")


def test_rejects_invalid_alignment_noncanonical_offsets_and_truncation(pk, tmp_path):
    """src/gguf.rs:3809-3837; a non-power-of-two multiple of 8 is a legal alignment (src/gguf.rs:3245-3263)."""
    seed = pk["seed"]
    align = lambda v: seed._kv("general.alignment", seed.T_U32, struct.pack("<I", v))
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=[align(3)]), "GGUF alignment 3 must be a multiple of 8 bytes")
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=[seed._kv("general.alignment", seed.T_U64, struct.pack("<Q", 32))]), "general.alignment must be U32")
    a, b = ("a", (1,), 0, f32s(1.0), 0), ("b", (1,), 0, f32s(2.0), 0)
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[a, b]), "tensor 'b' has non-canonical offset 0, expected 32")
    whole = raw_gguf(seed, tensors=[a])
    refused_bytes(pk, tmp_path, whole[:-32], "past file length")
    # alignment 24: accepted by the container parser (the refusal that follows is the family audit's, not the container's)
    ok = raw_gguf(seed, metas=[align(24)], tensors=[("a", (1,), 0, f32s(1.0), None), ("b", (1,), 0, f32s(2.0), None)], align=24)
    refused_bytes(pk, tmp_path, ok, "general.architecture")


def test_rejects_unsupported_tensor_types_and_shape_overflow(pk, tmp_path):
    """src/gguf.rs:3839-3861 and byte_len's rules (src/gguf.rs:427-451)."""
    seed = pk["seed"]
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[("q4_1", (32,), 3, b"\0" * 20, None)]), "unsupported GGML tensor type 3; this runtime currently supports")
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[("huge", (2 ** 63 - 1, 4), 0, b"", None)]), "tensor 'huge' element count overflow")
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[("huge", (2 ** 64 - 1, 2), 0, b"", None)]), "tensor 'huge' dimension does not fit usize")
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[("zero", (0,), 0, b"", None)]), "tensor 'zero' has a zero-sized dimension")
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[("ragged", (100,), 12, b"", None)]), "tensor 'ragged' row width 100 is not divisible by Q4K block size 256")
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[("odd", (96,), 6, b"\0" * 66, None)]), "require paired 32-element blocks (a multiple of 64)")
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[("r5", (1, 1, 1, 1, 1), 0, f32s(1.0), None)]), "tensor 'r5' has rank 5; supported ranks are 1..=4")
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[("n" * 64, (1,), 0, f32s(1.0), None)]), "is 64 bytes; maximum is 63")


def test_bounded_strings_arrays_and_keys(pk, tmp_path):
    """src/gguf.rs:2040-2052,2266-2292,2326-2345,3166-3203: a length word cannot make the parser reserve what the file does not
    hold, and the decoded metadata is charged against one cumulative budget."""
    seed = pk["seed"]
    T_ARRAY, T_STR = 9, seed.T_STR
    huge_string = struct.pack("<Q", 1 << 40)
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=[seed._s("k") + struct.pack("<I", T_STR) + huge_string]), "GGUF string length 1099511627776 exceeds limit 16777216")
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=[seed._s("k") + struct.pack("<I", T_STR) + struct.pack("<Q", 1000)]), "GGUF string length 1000 exceeds 0 remaining bytes")
    big_array = struct.pack("<IQ", seed.T_U32, 1 << 30)
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=[seed._kv("k", T_ARRAY, big_array)]), "GGUF array element count 1073741824 exceeds limit 1048576")
    short_array = struct.pack("<IQ", seed.T_U32, 1000)
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=[seed._kv("k", T_ARRAY, short_array)]), "needs at least 4000 bytes, but only 0 remain")
    for key, why in (("Upper.case", "is not a dot-separated lowercase identifier"), ("a..b", "is not a dot-separated lowercase identifier"),
                     ("", "GGUF metadata key cannot be empty"), ("caf\u00e9", "is not ASCII")):
        refused_bytes(pk, tmp_path, raw_gguf(seed, metas=[seed._kv(key, seed.T_U32, struct.pack("<I", 1))]), why)
    # seventeen strings of 16 MiB each pass their own limit and break the cumulative 256 MiB budget
    one = struct.pack("<Q", 16 << 20) + b"a" * (16 << 20)
    metas = [seed._s(f"s{i}") + struct.pack("<I", T_STR) + one for i in range(17)]
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=metas), "GGUF decoded allocation budget exceeded while reserving string storage")


def test_a_fifo_is_refused_without_blocking(pk, tmp_path):
    """src/gguf.rs:3073-3098."""
    import os
    path = tmp_path / "pipe.gguf"
    os.mkfifo(path)
    with pytest.raises(pk["capi"].MkError, match="is not a regular file"):
        pk["eng"].Model.inspect_gguf(path)


def test_quantised_rows_must_be_whole_blocks_and_need_the_quantisation_version(pk, tmp_path):
    """src/gguf.rs:4279-4326."""
    seed = pk["seed"]
    version = [seed._kv("general.quantization_version", seed.T_U32, struct.pack("<I", 2))]
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=version, tensors=[("q8", (16, 2), 8, b"\\0" * 34, None)]), "row width 16")
    for name, tag, nbytes in (("q2k", 10, 84), ("q3k", 11, 110), ("q4k", 12, 144)):
        refused_bytes(pk, tmp_path, raw_gguf(seed, metas=version, tensors=[(name, (128, 2), tag, b"\\0" * nbytes, None)]), "row width 128")
    for name, tag, block in (("q5_0", 6, 22), ("q5_1", 7, 24)):
        refused_bytes(pk, tmp_path, raw_gguf(seed, metas=version, tensors=[(name, (32, 2), tag, b"\\0" * block * 2, None)]), "paired 32-element blocks")
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[("q8", (32,), 8, b"\\0" * 34, None)]), "require general.quantization_version")


def test_rejects_noncanonical_keys_names_ranks_and_extents(pk, tmp_path):
    """src/gguf.rs:4397-4432."""
    seed = pk["seed"]
    refused_bytes(pk, tmp_path, raw_gguf(seed, metas=[seed._kv("Bad-Key", seed.T_U32, struct.pack("<I", 1))]), "dot-separated lowercase identifier")
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[("a" * 64, (1,), 0, f32s(1.0), None)]), "maximum is 63")
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[("scalar", (), 0, f32s(1.0), None)]), "supported ranks")
    refused_bytes(pk, tmp_path, raw_gguf(seed, tensors=[("empty", (0,), 0, b"", None)]), "zero-sized dimension")
