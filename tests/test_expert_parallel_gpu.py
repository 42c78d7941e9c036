"""Expert parallelism of the sparse-MoE family over two and four GPUs (one process per GPU).  Two forms:
replicated lanes - all ranks run the same ragged batches on their share of the experts and must end every forward with
the same bits; against the same checkpoint served from one GPU the schedule is identical and the logits differ only by
the association of the per-token sum over experts;
data-parallel lanes - every rank serves its own requests, the routed rows travel to the experts' ranks and back, and
every rank's results equal those of one GPU serving that rank's requests alone.
Needs as many CUDA devices as ranks; NVLS is off and the exchange kernels use plain peer stores."""
import importlib
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent

PROMPT_SEED, N_PROMPTS, NEW_TOKENS = 5, 5, 6
ENGINE_KW = dict(max_active_sequences=4, scheduler_token_budget=96, prefill_token_quantum=48, queue_capacity=16)


def make_prompts(vocab):
    rng = np.random.default_rng(PROMPT_SEED)
    return [rng.integers(0, vocab, int(n)).tolist() for n in rng.integers(3, 70, N_PROMPTS)]


def serve(eng, model, vocab):
    e = eng.Engine(model, record_logits=True, **ENGINE_KW)
    ids = e.submit([eng.Request(p, NEW_TOKENS) for p in make_prompts(vocab)], atomic_batch=False)
    e.run()
    return (e.trace(), [list(map(int, e.result(i)["tokens"])) for i in ids], [np.asarray(e.logits(i), dtype=np.float32) for i in ids])


CHILD = textwrap.dedent("""
    import importlib, pickle, sys, time
    sys.path.insert(0, %r)
    sys.path.insert(0, %r)
    import __graft_entry__ as entry
    entry.load_package()
    eng = importlib.import_module("macllm_infer_b200.engine")
    import test_expert_parallel_gpu as t
    rank, size, gguf, id_file, out_file, vocab = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], sys.argv[5], int(sys.argv[6])
    model = eng.Model.load_gguf(gguf, device=rank, kv_dtype="f32", matmul_path=1, max_batch_tokens=256, max_batch_lanes=8,
                                kv_capacity_tokens=2048, ep_rank=rank, ep_size=size)
    if rank == 0:
        uid = eng.Model.ep_unique_id()
        with open(id_file + ".tmp", "wb") as f:
            f.write(uid)
        import os
        os.replace(id_file + ".tmp", id_file)
    else:
        import os
        deadline = time.time() + 120
        while not os.path.exists(id_file):
            if time.time() > deadline:
                raise SystemExit("rank 0 never published the group id")
            time.sleep(0.05)
        uid = open(id_file, "rb").read()
    model.ep_init(uid)
    trace, tokens, logits = t.serve(eng, model, vocab)
    with open(out_file, "wb") as f:
        pickle.dump(dict(trace=trace, tokens=tokens, logits=logits, weight_bytes=model.spec().weight_bytes,
                         launches=model.launch_count()), f)
""") % (str(ROOT), str(ROOT / "tests"))


@pytest.mark.parametrize("ranks", [2, 4])
@pytest.mark.parametrize("exchange", ["fused", "nccl"])
def test_ranks_hold_their_share_of_the_experts_and_agree(mk, tmp_path, exchange, ranks):
    """exchange = fused: one kernel combines this rank's experts, stores the partial rows into the peers' memory over
    NVLink and adds all ranks' rows; nccl: combine kernel, ncclAllGather, sum kernel."""
    import pickle
    capi = importlib.import_module("macllm_infer_b200._capi")
    eng = importlib.import_module("macllm_infer_b200.engine")
    seed = importlib.import_module("macllm_infer_b200.seed_gguf")
    if capi.lib().mk_device_count() < ranks:
        pytest.skip(f"needs {ranks} CUDA devices")
    spec = seed.scaled("qwen3-30b-a3b", layers=2, vocab=2048, hidden=1024, experts=16)
    gguf = tmp_path / "moe.gguf"
    seed.write_seed_gguf(gguf, spec, seed=0)

    whole = eng.Model.load_gguf(gguf, device=0, kv_dtype="f32", matmul_path=1, max_batch_tokens=256, max_batch_lanes=8,
                                kv_capacity_tokens=2048)
    ref_trace, ref_tokens, ref_logits = serve(eng, whole, spec.vocab)
    whole_bytes = whole.spec().weight_bytes
    whole_launches = whole.launch_count()
    del whole

    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MACLLM_B200_EP_FUSED="1" if exchange == "fused" else "0")
    procs = [subprocess.Popen([sys.executable, "-c", CHILD, str(r), str(ranks), str(gguf), str(tmp_path / "ep.id"), str(tmp_path / f"out{r}.pkl"),
                               str(spec.vocab)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(ranks)]
    try:
        for p in procs:
            _, err = p.communicate(timeout=300)
            assert p.returncode == 0, err[-3000:]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    out = [pickle.load(open(tmp_path / f"out{r}.pkl", "rb")) for r in range(ranks)]

    # all ranks: the same schedule, tokens and logit bits
    for o in out[1:]:
        assert out[0]["trace"] == o["trace"] == ref_trace
        assert out[0]["tokens"] == o["tokens"]
        for a, b in zip(out[0]["logits"], o["logits"]):
            assert np.array_equal(a, b)
    # the fused exchange adds no launch to the single-GPU sequence; the NCCL form adds two per MoE layer and forward
    moe_layer_forwards = spec.layers * len(ref_trace)
    extra = 0 if exchange == "fused" else 2 * moe_layer_forwards
    assert all(o["launches"] == whole_launches + extra for o in out)
    # each rank holds its share of the expert banks
    expert_bytes = sum(seed._tensor_bytes(dims, qtype) for name, dims, qtype, _ in seed.tensor_plan(spec) if "_exps" in name)
    assert all(o["weight_bytes"] == whole_bytes - expert_bytes * (ranks - 1) // ranks for o in out)
    # against one GPU: rows computed from the same inputs agree up to the reassociated expert sum
    worst = 0.0
    for toks, lg, rtoks, rlg in zip(out[0]["tokens"], out[0]["logits"], ref_tokens, ref_logits):
        same = 0
        while same < min(len(toks), len(rtoks)) and toks[same] == rtoks[same]:
            same += 1
        rows = min(same + 1, len(lg), len(rlg))
        worst = max(worst, float(np.abs(lg[:rows] - rlg[:rows]).max()))
        if same < len(rtoks):
            top2 = np.sort(rlg[same])[-2:]
            assert top2[1] - top2[0] <= 2 * max(worst, 1e-3)
    assert worst <= 2e-2, worst


DP_ENGINE_KW = dict(max_active_sequences=4, scheduler_token_budget=96, prefill_token_quantum=48, queue_capacity=16)
DP_MODEL_KW = dict(kv_dtype="f16", matmul_path=0, max_batch_tokens=256, max_batch_lanes=8, kv_capacity_tokens=2048)


def dp_prompts(vocab, rank):
    """Ranks get different numbers of requests, so some of them run out of lanes first and tick idle."""
    rng = np.random.default_rng(PROMPT_SEED + 17 * rank)
    return [rng.integers(0, vocab, int(n)).tolist() for n in rng.integers(3, 70, 2 + (3 * rank + 3) % 5)]


def dp_collect(e, ids):
    return ([list(map(int, e.result(i)["tokens"])) for i in ids], [np.asarray(e.logits(i), dtype=np.float32) for i in ids])


DP_CHILD = textwrap.dedent("""
    import importlib, pickle, sys
    sys.path.insert(0, %r)
    sys.path.insert(0, %r)
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    eng = importlib.import_module("macllm_infer_b200.engine")
    import test_expert_parallel_gpu as t
    rank, size, gguf, port, out_file, vocab = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], int(sys.argv[4]), sys.argv[5], int(sys.argv[6])
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%%d" %% port, rank=rank, world_size=size)
    model = eng.Model.load_gguf(gguf, device=rank, ep_rank=rank, ep_size=size, ep_mode=1, **t.DP_MODEL_KW)
    box = [eng.Model.ep_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    model.ep_init(box[0])

    def total(n):
        v = torch.tensor([int(n)], dtype=torch.int64)
        dist.all_reduce(v)
        return int(v.item())

    e = eng.Engine(model, record_logits=True, **t.DP_ENGINE_KW)
    ids = e.submit([eng.Request(p, t.NEW_TOKENS) for p in t.dp_prompts(vocab, rank)], atomic_batch=False)
    ticks = eng.run_expert_parallel(e, model, total)
    tokens, logits = t.dp_collect(e, ids)
    with open(out_file, "wb") as f:
        pickle.dump(dict(tokens=tokens, logits=logits, trace=e.trace(), ticks=ticks, weight_bytes=model.spec().weight_bytes), f)
    dist.barrier()
    dist.destroy_process_group()
""") % (str(ROOT), str(ROOT / "tests"))


@pytest.mark.parametrize("ranks", [2, 4])
def test_data_parallel_lanes_with_dispatched_experts_match_one_gpu(mk, tmp_path, monkeypatch, ranks):
    """Every rank serves its own requests; each MoE layer sends the routed rows to the ranks that hold the experts and the
    outputs back.  The expert arithmetic of a row does not depend on where it runs or on which rows share its launch, so
    every rank must reproduce, bit for bit, what one GPU with all experts computes for that rank's requests."""
    import pickle
    import socket
    capi = importlib.import_module("macllm_infer_b200._capi")
    eng = importlib.import_module("macllm_infer_b200.engine")
    seed = importlib.import_module("macllm_infer_b200.seed_gguf")
    if capi.lib().mk_device_count() < ranks:
        pytest.skip(f"needs {ranks} CUDA devices")
    # the same matmul kernels at every width on both sides (the streamed blocks from one row up)
    monkeypatch.setenv("MACLLM_B200_STREAM_MIN_ROWS", "1")
    spec = seed.scaled("qwen3-30b-a3b", layers=2, vocab=2048, hidden=1024, experts=16)
    gguf = tmp_path / "moe.gguf"
    seed.write_seed_gguf(gguf, spec, seed=0)

    whole = eng.Model.load_gguf(gguf, device=0, **DP_MODEL_KW)
    want = []
    for r in range(ranks):
        e = eng.Engine(whole, record_logits=True, **DP_ENGINE_KW)
        ids = e.submit([eng.Request(p, NEW_TOKENS) for p in dp_prompts(spec.vocab, r)], atomic_batch=False)
        e.run()
        want.append(dp_collect(e, ids) + (e.trace(),))
        e.close()
    whole_bytes = whole.spec().weight_bytes
    del whole

    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MACLLM_B200_STREAM_MIN_ROWS="1")
    procs = [subprocess.Popen([sys.executable, "-c", DP_CHILD, str(r), str(ranks), str(gguf), str(port), str(tmp_path / f"dp{r}.pkl"), str(spec.vocab)],
                              env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(ranks)]
    try:
        for p in procs:
            _, err = p.communicate(timeout=300)
            assert p.returncode == 0, err[-3000:]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    out = [pickle.load(open(tmp_path / f"dp{r}.pkl", "rb")) for r in range(ranks)]
    # lock step: every rank took the same number of ticks, and the ranks with fewer ticks of their own idled the rest
    assert len({o["ticks"] for o in out}) == 1
    assert out[0]["ticks"] == max(len(w[2]) for w in want)
    assert min(len(o["trace"]) for o in out) < out[0]["ticks"]
    expert_bytes = sum(seed._tensor_bytes(dims, qtype) for name, dims, qtype, _ in seed.tensor_plan(spec) if "_exps" in name)
    assert all(o["weight_bytes"] == whole_bytes - expert_bytes * (ranks - 1) // ranks for o in out)
    for r, (o, (tokens, logits, trace)) in enumerate(zip(out, want)):
        assert o["trace"] == trace, r
        assert o["tokens"] == tokens, r
        for a, b in zip(o["logits"], logits):
            assert np.array_equal(a, b), (r, float(np.abs(a - b).max()))
