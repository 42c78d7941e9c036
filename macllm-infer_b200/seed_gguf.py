"""Synthetic GGUF checkpoints ("seed models") for the benchmark configurations.

Weights are N(0, 0.02) from a counter-based generator keyed by (seed, tensor name), quantised in a
Q4_K_M-shaped mix (Q4_K for every matrix except attn_v and the output matrix, which are Q6_K; norms
and the MoE router F32), and written as GGUF v3 with the metadata keys and tensor names the
reference's loader expects (src/gguf.rs:1768-1832, src/gguf_model.rs:65-194).  Both the B200 library
and the CPU oracle read the file this writes.
"""
from __future__ import annotations

import struct
import zlib
from dataclasses import dataclass, field, replace
from pathlib import Path

import numpy as np

from . import _capi as capi
from . import ops

F32, F16, Q8_0, Q4_K, Q6_K = capi.TYPE_F32, capi.TYPE_F16, capi.TYPE_Q8_0, capi.TYPE_Q4_K, capi.TYPE_Q6_K
GGUF_MAGIC = 0x46554747
ALIGN = 32
# GGUF metadata value type codes
T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64 = 4, 5, 6, 7, 8, 9, 10


@dataclass
class SeedSpec:
    arch: str
    layers: int
    hidden: int
    q_heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    context: int = 8192
    theta: float = 10000.0
    eps: float = 1e-5
    tied: bool = False
    experts: int = 0
    experts_used: int = 0
    expert_ffn: int = 0
    window: int = 4096
    attn_softcap: float = 50.0
    final_softcap: float = 30.0
    matrix_type: int = Q4_K      # the "everything else" type of the mix
    high_type: int = Q6_K        # attn_v and the output matrix
    name: str = "seed"
    extra: dict = field(default_factory=dict)


# The five benchmark shapes and scaled-down siblings for parity tests.
CONFIGS = {
    "tinyllama-1.1b": SeedSpec("llama", 22, 2048, 32, 4, 64, 5632, 32000, context=2048, theta=10000.0, eps=1e-5),
    "smollm3-3b": SeedSpec("smollm3", 36, 2048, 16, 4, 128, 11008, 128256, context=65536, theta=5e6, eps=1e-6, tied=True),
    "qwen3-8b": SeedSpec("qwen3", 36, 4096, 32, 8, 128, 12288, 151936, context=40960, theta=1e6, eps=1e-6),
    # context 16384 rather than Gemma 2's 8192: the benchmark's prompts reach 8192 tokens and 256 more are generated
    "gemma2-9b": SeedSpec("gemma2", 42, 3584, 16, 8, 256, 14336, 256000, context=16384, theta=10000.0, eps=1e-6, tied=True),
    "qwen3-30b-a3b": SeedSpec("qwen3moe", 48, 2048, 32, 4, 128, 6144, 151936, context=40960, theta=1e6, eps=1e-6,
                              experts=128, experts_used=8, expert_ffn=768),
}


def scaled(name: str, *, layers: int, vocab: int | None = None, hidden: int | None = None, ffn: int | None = None,
           experts: int | None = None, **kw) -> SeedSpec:
    """A smaller model of the same family and head geometry (for tests the CPU oracle finishes quickly)."""
    base = CONFIGS[name]
    spec = replace(base, layers=layers, **kw)
    if vocab is not None:
        spec.vocab = vocab
    if hidden is not None:
        spec.hidden = hidden
    if ffn is not None:
        spec.ffn = ffn
    if experts is not None:
        spec.experts = experts
    if spec.arch == "smollm3" and layers != 36:
        spec.extra = dict(spec.extra, **{"macllm.allow_scaled_layers": True})
    return spec


def _s(b: str) -> bytes:
    e = b.encode("utf-8")
    return struct.pack("<Q", len(e)) + e


def _kv(key: str, vtype: int, payload: bytes) -> bytes:
    return _s(key) + struct.pack("<I", vtype) + payload


def _meta(spec: SeedSpec) -> list[bytes]:
    a = spec.arch
    out = [
        _kv("general.architecture", T_STR, _s(a)),
        _kv("general.name", T_STR, _s(spec.name)),
        _kv("general.alignment", T_U32, struct.pack("<I", ALIGN)),
        _kv("general.quantization_version", T_U32, struct.pack("<I", 2)),  # required beside quantised tensors (src/gguf.rs:1019-1037)
        _kv(f"{a}.block_count", T_U32, struct.pack("<I", spec.layers)),
        _kv(f"{a}.context_length", T_U32, struct.pack("<I", spec.context)),
        _kv(f"{a}.embedding_length", T_U32, struct.pack("<I", spec.hidden)),
        _kv(f"{a}.feed_forward_length", T_U32, struct.pack("<I", spec.ffn)),
        _kv(f"{a}.attention.head_count", T_U32, struct.pack("<I", spec.q_heads)),
        _kv(f"{a}.attention.head_count_kv", T_U32, struct.pack("<I", spec.kv_heads)),
        _kv(f"{a}.attention.key_length", T_U32, struct.pack("<I", spec.head_dim)),
        _kv(f"{a}.attention.value_length", T_U32, struct.pack("<I", spec.head_dim)),
        _kv(f"{a}.attention.layer_norm_rms_epsilon", T_F32, struct.pack("<f", spec.eps)),
        _kv(f"{a}.rope.freq_base", T_F32, struct.pack("<f", spec.theta)),
        _kv(f"{a}.vocab_size", T_U32, struct.pack("<I", spec.vocab)),
    ]
    if a != "gemma2":
        out.append(_kv(f"{a}.rope.dimension_count", T_U32, struct.pack("<I", spec.head_dim)))
    if a == "gemma2":
        out += [
            _kv("gemma2.attention.sliding_window", T_U32, struct.pack("<I", spec.window)),
            _kv("gemma2.attn_logit_softcapping", T_F32, struct.pack("<f", spec.attn_softcap)),
            _kv("gemma2.final_logit_softcapping", T_F32, struct.pack("<f", spec.final_softcap)),
        ]
    if a == "qwen3moe":
        out += [
            _kv("qwen3moe.expert_count", T_U32, struct.pack("<I", spec.experts)),
            _kv("qwen3moe.expert_used_count", T_U32, struct.pack("<I", spec.experts_used)),
            _kv("qwen3moe.expert_feed_forward_length", T_U32, struct.pack("<I", spec.expert_ffn)),
        ]
    for k, v in spec.extra.items():
        if k != "rope_factors":  # a tensor's payload, not a metadata key (see tensor_plan)
            out.append(_kv(k, T_BOOL, struct.pack("<B", 1 if v else 0)))
    # a minimal embedded tokenizer: the reference's loader requires these keys (gguf_model.rs:3233-3262)
    toks = b"".join(_s(f"t{i}") for i in range(spec.vocab))
    out += [
        _kv("tokenizer.ggml.model", T_STR, _s("gpt2")),
        _kv("tokenizer.ggml.pre", T_STR, _s("default")),
        _kv("tokenizer.ggml.tokens", T_ARR, struct.pack("<IQ", T_STR, spec.vocab) + toks),
        _kv("tokenizer.ggml.token_type", T_ARR, struct.pack("<IQ", T_I32, spec.vocab) + np.ones(spec.vocab, np.int32).tobytes()),
        _kv("tokenizer.ggml.merges", T_ARR, struct.pack("<IQ", T_STR, 0)),
        _kv("tokenizer.ggml.eos_token_id", T_U32, struct.pack("<I", 2)),
        _kv("tokenizer.ggml.bos_token_id", T_U32, struct.pack("<I", 1)),
    ]
    return out


def tensor_plan(spec: SeedSpec) -> list[tuple[str, tuple[int, ...], int, float]]:
    """(name, logical dims outermost-first, ggml type, std or 0 for all-ones) in file order."""
    H, AW, KW = spec.hidden, spec.q_heads * spec.head_dim, spec.kv_heads * spec.head_dim
    m, hi = spec.matrix_type, spec.high_type
    t: list[tuple[str, tuple[int, ...], int, float]] = []
    t.append(("token_embd.weight", (spec.vocab, H), hi if spec.tied else m, 0.02))
    for l in range(spec.layers):
        p = f"blk.{l}."
        t.append((p + "attn_norm.weight", (H,), F32, 0.0))
        t.append((p + "attn_q.weight", (AW, H), m, 0.02))
        t.append((p + "attn_k.weight", (KW, H), m, 0.02))
        t.append((p + "attn_v.weight", (KW, H), hi, 0.02))
        t.append((p + "attn_output.weight", (H, AW), m, 0.02))
        if spec.arch in ("qwen3", "qwen3moe"):
            t.append((p + "attn_q_norm.weight", (spec.head_dim,), F32, 0.0))
            t.append((p + "attn_k_norm.weight", (spec.head_dim,), F32, 0.0))
        if spec.arch == "gemma2":
            t.append((p + "post_attention_norm.weight", (H,), F32, 0.0))
        t.append((p + "ffn_norm.weight", (H,), F32, 0.0))
        if spec.arch == "qwen3moe":
            E, F = spec.experts, spec.expert_ffn
            t.append((p + "ffn_gate_inp.weight", (E, H), F32, 1.0 / float(np.sqrt(H))))
            t.append((p + "ffn_gate_exps.weight", (E, F, H), m, 0.02))
            t.append((p + "ffn_up_exps.weight", (E, F, H), m, 0.02))
            t.append((p + "ffn_down_exps.weight", (E, H, F), m, 0.02))
        else:
            t.append((p + "ffn_gate.weight", (spec.ffn, H), m, 0.02))
            t.append((p + "ffn_up.weight", (spec.ffn, H), m, 0.02))
            t.append((p + "ffn_down.weight", (H, spec.ffn), m, 0.02))
        if spec.arch == "gemma2":
            t.append((p + "post_ffw_norm.weight", (H,), F32, 0.0))
    if spec.extra.get("rope_factors") is not None:
        t.append(("rope_freqs.weight", (len(spec.extra["rope_factors"]),), F32, -1.0))  # payload from spec.extra
    t.append(("output_norm.weight", (H,), F32, 0.0))
    if not spec.tied:
        t.append(("output.weight", (spec.vocab, H), hi, 0.02))
    return t


def _tensor_bytes(dims: tuple[int, ...], qtype: int) -> int:
    cols = dims[-1]
    rows = int(np.prod(dims[:-1])) if len(dims) > 1 else 1
    return rows * ops.row_bytes(qtype, cols)


def stream_of(name: str) -> int:
    return zlib.crc32(name.encode("utf-8")) & 0xFFFFFFFF


def _write_file(path: Path, metas: list[bytes], plan, spec: SeedSpec, seed: int) -> Path:
    """One GGUF file holding the given metadata records and the tensors of `plan` with their seeded payloads."""
    header = struct.pack("<IIQQ", GGUF_MAGIC, 3, len(plan), len(metas)) + b"".join(metas)
    infos = []
    offset = 0
    offsets = []
    for name, dims, qtype, _ in plan:
        offsets.append(offset)
        infos.append(_s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in reversed(dims)) +
                     struct.pack("<IQ", qtype, offset))
        offset += (_tensor_bytes(dims, qtype) + ALIGN - 1) // ALIGN * ALIGN
    head = header + b"".join(infos)
    pad = (-len(head)) % ALIGN
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        for (name, dims, qtype, std), off in zip(plan, offsets):
            n = _tensor_bytes(dims, qtype)
            if name == "rope_freqs.weight":
                data = np.asarray(spec.extra["rope_factors"], dtype=np.float32).tobytes()
            elif std == 0.0:
                data = np.ones(int(np.prod(dims)), dtype=np.float32).tobytes()
            else:
                cols = dims[-1]
                rows = int(np.prod(dims[:-1]))
                data = ops.seed_tensor(seed, stream_of(name), std, qtype, rows, cols).tobytes()
            assert len(data) == n, (name, len(data), n)
            f.write(data)
            f.write(b"\0" * ((-n) % ALIGN))
    return path


def write_seed_gguf(path: str | Path, spec: SeedSpec, seed: int = 0) -> Path:
    """Write the checkpoint; returns the path.  Deterministic in (spec, seed)."""
    return _write_file(Path(path), _meta(spec), tensor_plan(spec), spec, seed)


T_U16 = 2


def split_metas(index: int, count: int, tensors: int) -> list[bytes]:
    """The split.* records of shard `index` (src/gguf.rs:52-54,956-993: UINT16 index and count, INT32 tensor total)."""
    return [_kv("split.no", T_U16, struct.pack("<H", index)), _kv("split.count", T_U16, struct.pack("<H", count)),
            _kv("split.tensors.count", T_I32, struct.pack("<i", tensors))]


def write_seed_gguf_shards(directory: str | Path, prefix: str, spec: SeedSpec, shards: int, seed: int = 0) -> Path:
    """The same checkpoint as write_seed_gguf cut into `shards` files `<prefix>-0000i-of-0000n.gguf`: the tensors in
    file order in contiguous groups, the whole metadata in the first file, the architecture and the split records in
    the others.  Returns the path of the first shard, which is the one to load."""
    directory = Path(directory)
    plan = tensor_plan(spec)
    per = -(-len(plan) // shards)
    first = None
    for i in range(shards):
        metas = (_meta(spec) if i == 0 else [_kv("general.architecture", T_STR, _s(spec.arch))]) + split_metas(i, shards, len(plan))
        path = _write_file(directory / f"{prefix}-{i + 1:05d}-of-{shards:05d}.gguf", metas, plan[i * per:(i + 1) * per], spec, seed)
        first = first or path
    return first


def weight_bytes(spec: SeedSpec) -> dict:
    """Algorithmic byte counts of the checkpoint: all matrices, and what one decode row touches."""
    total = per_token = all_experts = experts_only = 0
    for name, dims, qtype, std in tensor_plan(spec):
        if len(dims) < 2:
            continue
        n = _tensor_bytes(dims, qtype)
        total += n
        if "_exps" in name:
            per_token += n // spec.experts * spec.experts_used
            all_experts += n
            experts_only += n
        elif name == "token_embd.weight" and not spec.tied:
            pass  # only a row gather touches it
        else:
            per_token += n
            all_experts += n
    kv_per_token = 2 * spec.layers * spec.kv_heads * spec.head_dim * 2
    # all_experts: what a decode tick touches once its lanes hit every expert (a batch of some 64 lanes and more)
    return {"total": total, "per_token": per_token, "all_experts": all_experts, "experts_only": experts_only, "kv_f16_per_token": kv_per_token}
