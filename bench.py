#!/usr/bin/env python
"""Benchmark of the continuous-batching step on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

Workload (default `smollm3-3b-ragged64`): a SmolLM3-3B-shaped decoder (36 layers, hidden 2048, 16 q /
4 kv heads, head_dim 128, FFN 11008, vocab 128256, NoPE every 4th layer, tied embeddings) with seeded
N(0, 0.02) weights written as a Q4_K_M-shaped GGUF, serving one ragged continuous batch of 64
sequences with prompt lengths uniform in [32, 1024], 512-token prefill chunks mixed with decode
(scheduler budget 2048 tokens per tick), 128 greedy decode tokens each, f16 paged KV in 16-token
blocks.  One "step" is that whole batch, admission to last token.  The metric is ragged-batch tokens/s
(prompt + generated tokens, whole job).

  value     tokens / summed device time of the ticks (CUDA events on the launching stream)
  e2e       tokens / wall time of the same steps through the engine's C ABI with host buffers: every
            tick copies its token ids and block tables host->device from pinned memory and reads the
            sampled tokens back
  roofline  the dominant kernel class of one extra profiled step (CUDA events around every launch)
  cpu_baseline  the CPU oracle (a port of the reference's CPU path) timed on a bounded sample

The other four workloads of the metric (`--workload`: tinyllama-1.1b-batch4, qwen3-8b-prefix32 with a shared prefix and
the prefix cache, gemma2-9b-long128, qwen3-30b-a3b-poisson with seeded Poisson arrivals) run the same way on their own
shapes; `--limit-requests` / `--new-tokens` cut slices of them.

N > 1 (torchrun): dense workloads run N independent replicas, one per GPU, each with its own request stream (the path
has no exchange step for them); the sparse-MoE workload runs expert parallelism with data-parallel lanes - every rank
serves its own requests and each MoE layer exchanges the routed rows (`config.ep`; `--ep off` for replicas).  The
reported time is the max over ranks.  `--http-clients N` adds a step through the `/completion` endpoint (`http` key),
`--microbench` prints the Q4_K matmul GB/s of the decode shapes instead.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

METRIC = "ragged-batch tokens/s (prefill+decode)"
UNIT = "tokens/s"

DEFAULT_WORKLOAD = "smollm3-3b-ragged64"
WORKLOAD_NAMES = ["tinyllama-1.1b-batch4", "smollm3-3b-ragged64", "qwen3-8b-prefix32", "gemma2-9b-long128", "qwen3-30b-a3b-poisson"]


# DRAM traffic of the dominant kernels relative to their algorithmic bytes, from one `ncu` capture each on the
# benchmark's shapes (dram__bytes_read.sum + dram__bytes_write.sum over the bytes counted here; profiles/).  The
# roofline block scales the live per-launch algorithmic bytes by these ratios.
NCU_TRAFFIC_RATIO = {
    "hgemm_tc": (98.8 + 21.4) / (90.2 + 8.4 + 45.1),      # gate|up with the activation in the epilogue: every operand once; part of the f16 output is still in L2 at kernel end
    "paged_attention": (77.0 + 1.9) / (72.4 + 4.2),
    "qstream_tc": (25.70 + 0.004) / (25.36 + 0.26),         # streamed gate|up of a decode tick: every weight block once, the partial sums stay in L2
}


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback")


def workloads_module():
    entry.load_package()
    return importlib.import_module("macllm_infer_b200.workloads")


def checkpoint_path(config: str) -> Path:
    d = Path(os.environ.get("MACLLM_SEED_DIR", tempfile.gettempdir())) / "macllm_b200_seed"
    d.mkdir(parents=True, exist_ok=True)
    return d / f"{config}.gguf"


def ensure_checkpoint(config: str) -> Path:
    seed = importlib.import_module("macllm_infer_b200.seed_gguf")
    path = checkpoint_path(config)
    done = path.with_suffix(".done")
    if not done.exists():
        t0 = time.time()
        seed.write_seed_gguf(path, seed.CONFIGS[config], seed=0)
        done.write_text("ok")
        print(f"[bench] wrote {path} ({path.stat().st_size / 1e9:.2f} GB) in {time.time() - t0:.1f}s", file=sys.stderr)
    return path


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None, reasons=sorted(reasons),
                    samples=len(sm))


def dist_setup(n_gpus: int, backend: str = "nccl"):
    """One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*).  Replicas share nothing on
    the data path; the process group only carries the barrier and the two scalar reductions of the report.
    backend "gloo" keeps everything on the CPU (used by the CPU tests of this plumbing)."""
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist_mod.init_process_group(backend)
        dist = dist_mod
    return rank, local, world, dist


def _on_gpu(dist) -> bool:
    return dist.get_backend() == "nccl"


def barrier(dist):
    if dist is not None:
        dist.barrier()
        if _on_gpu(dist):
            import torch
            torch.cuda.synchronize()


def _all_reduce(dist, x: float, op_name: str) -> float:
    if dist is None:
        return x
    import torch
    t = torch.tensor([x], dtype=torch.float64, device="cuda" if _on_gpu(dist) else "cpu")
    dist.all_reduce(t, op=getattr(dist.ReduceOp, op_name))
    return float(t.item())


def all_max(dist, x: float) -> float:
    return _all_reduce(dist, x, "MAX")


def all_sum(dist, x: float) -> float:
    return _all_reduce(dist, x, "SUM")


def aggregate(dist, tokens: float, seconds: float) -> tuple[float, float, float]:
    """Whole-job figures of N replicas: (tokens of all ranks, slowest rank's time, tokens / that time)."""
    total = all_sum(dist, float(tokens))
    slowest = all_max(dist, float(seconds))
    return total, slowest, total / max(slowest, 1e-12)


def make_lockstep(dist):
    """The per-tick agreement of an expert-parallel group: (sum of the ranks' outstanding requests, did any rank fail)."""
    import torch

    def lockstep(n, failed=False):
        t = torch.tensor([float(n), 1.0 if failed else 0.0], dtype=torch.float64, device="cuda" if _on_gpu(dist) else "cpu")
        dist.all_reduce(t)
        return int(round(float(t[0].item()))), float(t[1].item()) > 0.0
    return lockstep


def new_engine(eng_mod, model, w, active: int, n_requests: int):
    return eng_mod.Engine(model, max_active_sequences=active, scheduler_token_budget=w.budget, prefill_token_quantum=w.quantum,
                          queue_capacity=n_requests + 8)


def drive(eng_mod, model, eng, w, reqs, lockstep=None):
    """Submits the requests the way the workload says and yields after every scheduler tick.
    - one atomic batch (configurations 1, 2, 4);
    - prefix reuse (configuration 3): request 0 alone until it has finished, then the others in submission order;
    - Poisson arrivals (configuration 5): a request is submitted once the step's clock has passed its arrival time; the
      clock is the wall time since the step began, and it jumps to the next arrival whenever the engine would idle, so
      that a step measures service, not waiting.
    lockstep (expert parallelism with data-parallel lanes): `lockstep(n, failed)` returns (sum of n over all ranks, whether
    any rank reported a failure).  Every rank then ticks until no rank has work left, and a rank with no lane to run takes
    the tick idle (it serves the others' rows).  An exception on one rank is held until the next sum, where every rank
    learns of it and all leave the loop in the same iteration - no rank is left waiting in a collective."""
    prompts, new, arrivals = reqs
    mk = lambda i: eng_mod.Request(prompts[i], new[i])
    ids = []
    drive.idle_s = 0.0
    if w.arrival_rate > 0:
        waves = None
    else:
        waves = [(0, 1, False), (1, len(prompts), False)] if w.shared_prefix else [(0, len(prompts), True)]
        waves = [x for x in waves if x[1] > x[0]]
    t0, skipped, nxt = time.perf_counter(), 0.0, 0
    failure = None
    while True:
        outstanding = (len(prompts) - nxt) + eng.pending()
        if lockstep is None:
            if outstanding <= 0:
                break
        else:
            total, any_failed = lockstep(outstanding, failure is not None)
            if any_failed:
                raise RuntimeError(failure or "another rank of the expert-parallel group failed")
            if total <= 0:
                break
        try:
            lanes, skipped, nxt = _tick(eng_mod, model, eng, reqs, mk, waves, ids, lockstep is not None, t0, skipped, nxt)
        except Exception as e:
            if lockstep is None:
                raise
            failure = f"{type(e).__name__}: {e}"
            continue
        yield lanes
    drive.last_ids = ids


def _tick(eng_mod, model, eng, reqs, mk, waves, ids, in_lockstep, t0, skipped, nxt):
    """One iteration of drive(): submit what is due (extending `ids`), run one scheduler tick or idle through it.
    Returns (lanes, skipped, nxt)."""
    prompts, _, arrivals = reqs
    if waves is None:
        now = time.perf_counter() - t0 + skipped
        if eng.pending() == 0 and nxt < len(prompts) and arrivals[nxt] > now:
            skipped += arrivals[nxt] - now
            now = arrivals[nxt]
        wave = []
        while nxt < len(prompts) and arrivals[nxt] <= now:
            wave.append(mk(nxt))
            nxt += 1
        if wave:
            ids.extend(eng.submit(wave))
    elif eng.pending() == 0 and waves:
        lo, hi, atomic = waves.pop(0)
        ids.extend(eng.submit([mk(i) for i in range(lo, hi)], atomic_batch=atomic))
        nxt = hi
    lanes = eng.step()
    if lanes == 0 and in_lockstep:
        t_idle = time.perf_counter()
        model.ep_idle_tick()
        model.synchronize()
        drive.idle_s += time.perf_counter() - t_idle
    return lanes, skipped, nxt


def run_step(eng_mod, model, w, reqs, active: int, lockstep=None):
    """One step: the whole workload through a fresh engine.  Returns (tokens, wall s, engine stats, prefix diagnostics).
    Under lock step the device time of the stats also counts the ticks this rank idled through (timed on the host around
    the idle exchange and a synchronize)."""
    prompts, new, _ = reqs
    eng = new_engine(eng_mod, model, w, active, len(prompts))
    model.synchronize()
    t0 = time.perf_counter()
    err = None
    try:
        for _ in drive(eng_mod, model, eng, w, reqs, lockstep):
            pass
        model.synchronize()
    except Exception as e:
        if lockstep is None:
            raise
        err = str(e)
    wall = time.perf_counter() - t0
    st = eng.stats()
    st["device_ms"] += drive.idle_s * 1e3
    toks = sum(len(p) for p in prompts)
    gen = 0
    for i in (drive.last_ids if err is None else []):
        r = eng.result(i)
        if r["state"] != "done":
            err = f"request {i} ended in state {r['state']}: {r['message']}"
            break
        gen += len(r["tokens"])
        toks -= r["cached_tokens"]          # prompt tokens served from the prefix cache were not computed
    st["generated_tokens"] = gen
    diag = model.prefix_diagnostics() if w.prefix_capacity_tokens and err is None else None
    eng.close()
    if lockstep is not None:
        # every rank of the group learns whether the step failed anywhere, so that all of them raise (or none does)
        _, any_failed = lockstep(0, err is not None)
        if any_failed:
            raise RuntimeError(err or "the step failed on another rank of the expert-parallel group")
    elif err is not None:
        raise RuntimeError(err)
    return toks + gen, wall, st, diag


def http_step(eng_mod, model, w, reqs, active: int, clients: int) -> dict:
    """The same workload through the raw `/completion` endpoint (macllm_infer_b200.server, the reference's benchmark
    surface src/server.rs:633-666) on 127.0.0.1: `clients` threads each post their share of the requests one after the
    other (non-streamed, token-id prompts) and the step ends with the last response - the reference's own throughput
    definition, total tokens / wall time from the first submission to the last completion (src/benchmark/serving.rs:301-328)."""
    import http.client
    import threading
    srv_mod = importlib.import_module("macllm_infer_b200.server")
    prompts, new, _ = reqs
    server = srv_mod.CompletionServer(lambda: (new_engine(eng_mod, model, w, active, len(prompts)), model)).start()
    done = [0] * clients
    errors = []

    def client(c):
        conn = http.client.HTTPConnection("127.0.0.1", server.port, timeout=600)
        for i in range(c, len(prompts), clients):
            body = {"prompt": [int(t) for t in prompts[i]], "n_predict": int(new[i]), "temperature": 0.0, "top_k": 1, "top_p": 1.0, "seed": 0,
                    "cache_prompt": True, "stream": False, "return_tokens": True, "id_slot": 0, "ignore_eos": True, "repeat_penalty": 1.0,
                    "response_fields": srv_mod.RAW_COMPLETION_RESPONSE_FIELDS}
            conn.request("POST", "/completion", body=json.dumps(body), headers={"Content-Type": "application/json"})
            r = conn.getresponse()
            out = json.loads(r.read())
            if r.status != 200:
                errors.append(out)
                return
            done[c] += out["tokens_predicted"] + out["timings/prompt_n"]
        conn.close()
    try:
        threads = [threading.Thread(target=client, args=(c,)) for c in range(clients)]
        t0 = time.perf_counter()
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        wall = time.perf_counter() - t0
    finally:
        server.stop()
    if errors:
        raise RuntimeError(f"/completion answered an error: {errors[0]}")
    return dict(value=sum(done) / wall, unit=UNIT, clients=clients, requests=len(prompts), wall_s=round(wall, 3),
                surface="POST /completion on 127.0.0.1, non-streamed, token-id prompts, one connection per client")


def tick_classes(eng_mod, model, w, reqs, active: int, weight_bytes_per_pass: float, kv_bytes_per_token: float, hbm_gbs: float,
                 window_layers: tuple = (0, 0, 0), lockstep=None) -> dict:
    """One more (untimed) step driven tick by tick: device time and algorithmic HBM bytes per tick class.
    A tick's algorithmic bytes = the weight bytes one pass touches + the K/V history its lanes attend to (sliding-window
    layers count at most `window` tokens); `hbm_frac` = those bytes / device time / measured copy bandwidth - the decode
    roofline of the metric."""
    prompts, new, _ = reqs
    eng = new_engine(eng_mod, model, w, active, len(prompts))
    ms = []
    before = model.launch_count()
    for lanes in drive(eng_mod, model, eng, w, reqs, lockstep):
        if lanes > 0 and model.launch_count() != before:  # a step that only delivers events runs no forward pass
            ms.append(model.last_forward_ms())
        before = model.launch_count()
    trace = eng.trace()
    eng.close()
    n_sliding, n_layers, window = window_layers
    out = {}
    for t, dev_ms in zip(trace, ms):
        toks = sum(n for _, _, n in t)
        if toks == 0:
            continue
        cls = "decode" if toks == len(t) else ("mixed" if any(n == 1 for _, _, n in t) else "prefill")
        kv = 0.0
        for _, sp, n in t:
            ctx = sp + n
            if n_sliding:
                kv += kv_bytes_per_token / n_layers * ((n_layers - n_sliding) * ctx + n_sliding * min(ctx, window + n))
            else:
                kv += kv_bytes_per_token * ctx
        a = out.setdefault(cls, dict(ticks=0, tokens=0, lanes=0, ms=0.0, bytes=0.0))
        a["ticks"] += 1
        a["tokens"] += toks
        a["lanes"] += len(t)
        a["ms"] += dev_ms
        a["bytes"] += weight_bytes_per_pass + kv
    for a in out.values():
        a["tokens_per_s"] = round(a["tokens"] / max(a["ms"], 1e-9) * 1e3, 1)
        a["ms_per_tick"] = round(a["ms"] / a["ticks"], 3)
        a["lanes_per_tick"] = round(a["lanes"] / a["ticks"], 1)
        a["gbs"] = round(a["bytes"] / max(a["ms"], 1e-9) / 1e6, 1)
        a["hbm_frac"] = round(a["bytes"] / max(a["ms"], 1e-9) / 1e6 / hbm_gbs, 4)
        a["ms"] = round(a["ms"], 2)
        del a["bytes"], a["lanes"]
    return out


Q4K_SHAPES = [(2048, 2048), (256, 2048), (5632, 2048), (2048, 5632), (11008, 2048), (2048, 11008), (12288, 4096), (24576, 4096), (4096, 12288)]


def microbench() -> None:
    """Q4_K matmul micro-benchmark: achieved GB/s on the algorithmic bytes of the matrix (rows * cols * 144/256) for
    the decode shapes of the first three configurations at 1, 4, 8, 16 and 64 activation rows: the integer GEMV (up to 8
    rows) and the streamed tensor-core kernel side by side.  Operands resident, L2 flushed before every launch, CUDA
    events around the launch.  One JSON line per shape."""
    ops = importlib.import_module("macllm_infer_b200.ops")
    capi = importlib.import_module("macllm_infer_b200._capi")
    pk = peaks()
    rng = np.random.default_rng(0)
    for rows, cols in Q4K_SHAPES:
        wq = ops.seed_tensor(0, 1, 0.02, capi.TYPE_Q4_K, rows, cols)
        nbytes = rows * cols * 144 // 256
        line = dict(kernel="q4k_matmul", rows=rows, cols=cols, weight_mb=round(nbytes / 1e6, 2), peak_gbs=pk["hbm_gbs"], peak_source=pk["source"])
        for T in (1, 4, 8, 16, 64):
            x = rng.standard_normal((T, cols)).astype(np.float32)
            for label, path in (("gemv", capi.PATH_GEMV), ("stream", capi.PATH_STREAM)):
                if label == "gemv" and T > 8:
                    continue
                ms = ops.qmatmul_time(capi.TYPE_Q4_K, wq, rows, cols, x, path, 20)
                line[f"T{T}_{label}"] = dict(us=round(ms * 1e3, 1), gbs=round(nbytes / ms / 1e6, 1), frac=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
        print(json.dumps(line), flush=True)


def cpu_model_name() -> str:
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown CPU"


def cpu_baseline(w, path, budget_s: float, threads: int) -> dict:
    """The oracle (a port of the reference's CPU path: no Rust toolchain here to build the reference itself) on a bounded
    sample of the same workload: the first S sequences with 4 new tokens each through the oracle's own scheduler with the
    workload's quantum and budget - prefill ticks, mixed ticks and at least three decode ticks - on `threads` OpenMP
    threads.  S is the largest number of sequences whose prompts fit the time budget at the rate of a short probe."""
    from oracle import decoder, engine as oe, mathlib
    mathlib.build()
    mathlib.set_num_threads(threads)
    wl = workloads_module()
    t0 = time.time()
    dec = decoder.Decoder(path, kv_dtype="f32", matmul_mode=1)
    load_s = time.time() - t0
    prompts, _, _ = wl.make_requests(w, dec.vocab, 0)
    # probe: a 16-token prefill
    om = oe.OracleModel(dec.vocab, dec.max_context, 16, 8, 1024, 0, decoder=dec)
    s = om.new_session()
    ids = [int(x) for x in prompts[0][:16]]
    t = time.time()
    om.forward([(s, ids, 0)], om.reserve_batch([(s, 0, len(ids))]))
    rate = len(ids) / max(time.time() - t, 1e-6)
    S, total = 0, 0
    order = sorted(range(len(prompts)), key=lambda i: len(prompts[i])) if w.shared_prefix == 0 else list(range(len(prompts)))
    chosen = []
    for i in order:
        if chosen and (total + len(prompts[i])) / rate > budget_s:
            break
        chosen.append(i)
        total += len(prompts[i])
        if len(chosen) >= 8:
            break
    sample = [[int(x) for x in prompts[i]] for i in chosen]
    if total / rate > 2.5 * budget_s:   # even one prompt is too long for the budget: its head
        keep = max(32, int(budget_s * rate))
        sample = [sample[0][:keep]]
    new = 4
    cap = sum(len(p) + new + 32 for p in sample)
    om = oe.OracleModel(dec.vocab, dec.max_context, 16, 8, cap, 0, decoder=dec)
    e = oe.OracleEngine(om, max_active_sequences=max(len(sample), 1), scheduler_token_budget=w.budget, prefill_token_quantum=w.quantum,
                        queue_capacity=len(sample) + 8)
    e.submit([oe.Req(p, new) for p in sample], atomic_batch=True)
    t = time.time()
    e.run()
    dt = time.time() - t
    ticks = e.trace
    decode_ticks = sum(1 for tk in ticks if all(n == 1 for _, _, n in tk))
    tokens = sum(len(p) for p in sample) + new * len(sample)
    return dict(value=tokens / dt, unit=UNIT, cores=mathlib.num_threads(), kind="port", cpu=cpu_model_name(),
                sample=f"the {len(sample)} shortest sequences of the workload ({sum(len(p) for p in sample)} prompt tokens), {new} new tokens each, "
                       f"quantum {w.quantum}, budget {w.budget}: {len(ticks)} ticks of which {decode_ticks} decode ticks, {dt:.1f}s "
                       f"(checkpoint load {load_s:.1f}s not counted)")


def q4k_gemv_block(hbm_gbs: float) -> dict:
    """The metric's second half: Q4_K matrix-vector products of the decode path at 1 and 8 activation rows on the gate/up
    shape of configuration 2 and the feed-forward shape of configuration 3, on the integer GEMV and on the streamed
    tensor-core kernel: achieved GB/s on the bytes of the matrix, operands resident, L2 flushed before every launch, CUDA
    events around the launch."""
    ops = importlib.import_module("macllm_infer_b200.ops")
    capi = importlib.import_module("macllm_infer_b200._capi")
    rng = np.random.default_rng(0)
    out = {}
    for rows, cols in ((11008, 2048), (12288, 4096)):
        wq = ops.seed_tensor(0, 1, 0.02, capi.TYPE_Q4_K, rows, cols)
        nbytes = rows * cols * 144 // 256
        for T in (1, 8):
            x = rng.standard_normal((T, cols)).astype(np.float32)
            ms = ops.qmatmul_time(capi.TYPE_Q4_K, wq, rows, cols, x, capi.PATH_GEMV, 10)
            out[f"{rows}x{cols}_T{T}"] = dict(us=round(ms * 1e3, 1), gbs=round(nbytes / ms / 1e6, 1), frac=round(nbytes / ms / 1e6 / hbm_gbs, 4))
            # the same product on the streamed tensor-core kernel, which is what a tick of 1..64 rows runs in automatic mode
            ms = ops.qmatmul_time(capi.TYPE_Q4_K, wq, rows, cols, x, capi.PATH_STREAM, 10)
            out[f"{rows}x{cols}_T{T}_streamed"] = dict(us=round(ms * 1e3, 1), gbs=round(nbytes / ms / 1e6, 1),
                                                      frac=round(nbytes / ms / 1e6 / hbm_gbs, 4))
    return out


def plan_arena(w, prompts, new, kv_per_token: int, kv_budget_gb: float):
    """(active sequences, KV arena tokens): the arena holds the active set at its longest; when that exceeds the budget the
    active set shrinks."""
    active = min(w.max_active(), len(prompts))

    def arena_tokens(a):
        longest = sorted(((len(p) + k + 31) // 16 * 16 + 16 for p, k in zip(prompts, new)), reverse=True)
        return sum(longest[:a]) + w.prefix_capacity_tokens
    while active > 1 and arena_tokens(active) * kv_per_token > kv_budget_gb * 1e9:
        active = active * 3 // 4
    return active, arena_tokens(active)


EP_SLICE_WORKLOAD = "qwen3-30b-a3b-poisson"
EP_SLICE_REQUESTS = 64
EP_SLICE_DEADLINE_S = 480.0   # one GPU takes about 100 s, most of it writing the 17 GB seeded checkpoint


def line_emitter(out):
    """Returns emit(ep=None): prints the JSON line once (the first call wins; later calls do nothing).  `out` is None on the
    ranks that print nothing."""
    lock = threading.Lock()
    done = []

    def emit(ep=None):
        with lock:
            if done:
                return False
            done.append(True)
            if out is not None:
                line = dict(out)
                if ep is not None:
                    line["ep"] = ep
                print(json.dumps(line), flush=True)
            return True
    return emit


def ep_slice(eng_mod, wl, seed, rank: int, local: int, world: int, dist, kv_budget_gb: float) -> dict:
    """The sparse-MoE workload's curve beside the headline: the first EP_SLICE_REQUESTS requests per rank of the Poisson
    workload on the full 48-layer, 128-expert shape, one warm-up step and one timed step.  One GPU serves them with every
    expert resident; N > 1 runs expert parallelism with data-parallel lanes over the same N ranks (each rank its own
    requests, the routed rows exchanged per MoE layer).  Every phase ends with an agreement over all ranks, so a failure on
    one rank makes all of them report it instead of leaving the others in a collective."""
    w = wl.WORKLOADS[EP_SLICE_WORKLOAD]
    spec = seed.CONFIGS[w.config]
    if spec.experts % world != 0:
        return dict(skipped=f"{spec.experts} experts do not split over {world} ranks")
    agree = make_lockstep(dist) if dist is not None else (lambda n, failed=False: (n, failed))

    def phase(fn):
        err, out = None, None
        try:
            out = fn()
        except Exception as e:
            err = f"{type(e).__name__}: {e}"
        if agree(0, err is not None)[1]:
            raise RuntimeError(err or "another rank failed")
        return out
    phase(lambda: ensure_checkpoint(w.config) if rank == 0 else None)
    path = checkpoint_path(w.config)
    reqs = wl.make_requests(w, spec.vocab, rank, EP_SLICE_REQUESTS)
    prompts, new, _ = reqs
    kv_per_token = 2 * spec.layers * spec.kv_heads * spec.head_dim * 2
    active, cap = plan_arena(w, prompts, new, kv_per_token, kv_budget_gb)
    ep_kw = dict(ep_rank=rank, ep_size=world, ep_mode=1) if world > 1 else {}
    model = phase(lambda: eng_mod.Model.load_gguf(path, device=local, kv_capacity_tokens=cap, kv_dtype="f16", max_batch_tokens=w.budget,
                                                  max_batch_lanes=active, **ep_kw))
    try:
        lockstep = None
        if world > 1:
            box = [eng_mod.Model.ep_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            phase(lambda: model.ep_init(box[0]))
            lockstep = agree
        run_step(eng_mod, model, w, reqs, active, lockstep)            # warm-up
        barrier(dist)
        tokens, wall, st, _ = run_step(eng_mod, model, w, reqs, active, lockstep)
        tokens_all = all_sum(dist, float(tokens))
        dev = all_max(dist, st["device_ms"] / 1e3)
        wall = all_max(dist, wall)
        return dict(workload=f"{EP_SLICE_WORKLOAD}, first {EP_SLICE_REQUESTS} requests per rank", ranks=world,
                    parallelism=f"dp{world} lanes x ep{world} experts" if world > 1 else "one GPU, all experts resident",
                    local_experts=spec.experts // world, value=tokens_all / max(dev, 1e-12), e2e=tokens_all / max(wall, 1e-12), unit=UNIT,
                    steps=1, warmup=1, ms_per_step=wall * 1e3, ticks_per_step=int(st["ticks"]), scaling="weak")
    finally:
        model.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=WORKLOAD_NAMES)
    ap.add_argument("--matmul-path", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    # a shorter slice of the same workload for profiler captures (a number printed by such a run is not a bench value)
    ap.add_argument("--new-tokens", type=int, default=0, help="override the generated tokens per sequence")
    ap.add_argument("--limit-requests", type=int, default=0, help="only the first N requests of the workload (per replica)")
    ap.add_argument("--kv-budget-gb", type=float, default=110.0, help="largest KV arena; the active set shrinks until it fits")
    ap.add_argument("--ep", default="auto", choices=["auto", "on", "off"],
                    help="N > 1 and a sparse-MoE workload: expert parallelism with data-parallel lanes (auto = on) instead of replicas")
    ap.add_argument("--http-clients", type=int, default=0,
                    help="also run one step through the /completion endpoint with this many concurrent clients (adds an `http` key)")
    ap.add_argument("--no-ep-slice", action="store_true",
                    help="default workload only: skip the slice of the sparse-MoE workload that adds the `ep` key (one GPU: all experts "
                         "resident; N > 1: expert parallelism over the same ranks)")
    ap.add_argument("--no-profiled-step", action="store_true", help="skip the extra step that times every launch")
    ap.add_argument("--microbench", action="store_true", help="Q4_K matmul GB/s on the decode shapes instead of the workload")
    args = ap.parse_args()

    rank, local, world, dist = dist_setup(args.gpus)
    wl = workloads_module()
    w = wl.WORKLOADS[args.workload]
    if args.new_tokens > 0:
        from dataclasses import replace
        w = replace(w, new_tokens=args.new_tokens)
    if rank == 0:
        entry.ensure_built()
    barrier(dist)
    seed = importlib.import_module("macllm_infer_b200.seed_gguf")
    spec = seed.CONFIGS[w.config]
    wb = seed.weight_bytes(spec)
    kv_per_token = 2 * spec.layers * spec.kv_heads * spec.head_dim * 2
    sliced = args.new_tokens > 0 or args.limit_requests > 0
    config = dict(workload=args.workload + (" (slice)" if sliced else ""), model_shape=w.config, requests_per_gpu=w.seqs if args.limit_requests <= 0 else min(w.seqs, args.limit_requests),
                  new_tokens=w.new_tokens, prefill_quantum=w.quantum, scheduler_token_budget=w.budget, kv="f16 paged, 16-token blocks",
                  quant="Q4_K_M-shaped GGUF (Q4_K, Q6_K for attn_v and output)", parallelism=f"replicas x{world}",
                  l2="inputs larger than L2 (weights %.2f GB per pass)" % (wb["per_token"] / 1e9))
    if w.shared_prefix:
        config.update(shared_prefix_tokens=w.shared_prefix, prefix_capacity_tokens=w.prefix_capacity_tokens)
    if w.arrival_rate:
        config.update(arrivals=f"Poisson {w.arrival_rate:g} requests/s, replayed from a seeded list; the clock skips idle time")

    if args.microbench:
        if rank == 0:
            microbench()
        return

    if args.impl == "reference":
        # The reference is Rust on candle and cannot be built here (no cargo/rustc): the reference arm is the CPU oracle,
        # the port of its CPU path, on a bounded sample per step, on every host core (rank 0 alone runs under torchrun,
        # which exports OMP_NUM_THREADS=1: the thread count is set explicitly).
        if rank != 0:
            return
        path = ensure_checkpoint(w.config)
        threads = os.cpu_count() or 1
        budget = max(4.0, 150.0 / max(args.steps + args.warmup, 1))
        vals = []
        for i in range(args.warmup + args.steps):
            b = cpu_baseline(w, path, budget, threads)
            if i >= args.warmup:
                vals.append(b)
        v = float(np.mean([b["value"] for b in vals])) if vals else 0.0
        b = vals[-1] if vals else dict(cores=0, sample="none", kind="port", cpu=cpu_model_name())
        out = dict(metric=METRIC, value=v, unit=UNIT, n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                   ms_per_step=None, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="int8 x int4/6 block dots, f32 accumulate",
                   data="synthetic", config=config, impl="reference",
                   cpu_baseline=dict(value=v, unit=UNIT, cores=b["cores"], kind=b["kind"], cpu=b["cpu"], sample=b["sample"]),
                   e2e=dict(value=v, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
        print(json.dumps(out))
        return

    ep = world > 1 and spec.experts > 0 and args.ep != "off"
    if args.ep == "on" and not ep:
        raise SystemExit("--ep on needs more than one GPU and a sparse-MoE workload")
    if ep:
        if spec.experts % world != 0:
            raise SystemExit(f"{spec.experts} experts do not split over {world} ranks")
        config["parallelism"] = f"dp{world} lanes x ep{world} experts"
        config["ep"] = dict(ranks=world, local_experts=spec.experts // world, lanes="data-parallel: every rank schedules its own requests",
                            exchange="per MoE layer: routed rows to the experts' ranks and outputs back, peer stores over NVLink",
                            lockstep="one scalar all-reduce per tick; a rank without lanes serves the others' rows")
    capi = importlib.import_module("macllm_infer_b200._capi")
    eng_mod = importlib.import_module("macllm_infer_b200.engine")
    if capi.lib().mk_device_count() <= 0:
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    if rank == 0:
        ensure_checkpoint(w.config)
    barrier(dist)
    path = checkpoint_path(w.config)

    reqs = wl.make_requests(w, spec.vocab, rank, args.limit_requests)
    prompts, new, _ = reqs
    active, cap = plan_arena(w, prompts, new, kv_per_token, args.kv_budget_gb)
    config.update(active_sequences=active, kv_arena_gb=round(cap * kv_per_token / 1e9, 2))
    model = eng_mod.Model.load_gguf(path, device=local, kv_capacity_tokens=cap, kv_dtype="f16", prefix_capacity_tokens=w.prefix_capacity_tokens,
                                    max_batch_tokens=w.budget, max_batch_lanes=active, matmul_path=args.matmul_path,
                                    **(dict(ep_rank=rank, ep_size=world, ep_mode=1) if ep else {}))
    lockstep = None
    if ep:
        box = [eng_mod.Model.ep_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        model.ep_init(box[0])
        lockstep = make_lockstep(dist)
    for _ in range(args.warmup):
        run_step(eng_mod, model, w, reqs, active, lockstep)
    sampler = ClockSampler(local)
    barrier(dist)
    if rank == 0:
        sampler.start()
    launches0 = model.launch_count()
    h2d0, d2h0 = model.transfer_bytes()
    tokens = 0
    generated = 0
    dev_ms = 0.0
    ticks = 0
    diag = None
    forward_kinds = dict(suffix_prefill_ms=0.0, first_token_ms=0.0, decode_ms=0.0, mixed_ms=0.0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        n, wall, st, diag = run_step(eng_mod, model, w, reqs, active, lockstep)
        tokens += n
        generated += st["generated_tokens"]
        dev_ms += st["device_ms"]
        ticks += st["ticks"]
        for k in forward_kinds:   # the engine's own split of the device time by whole-forward kind (src/engine.rs:430-439,601-619)
            forward_kinds[k] += float(st.get(k, 0.0))
    barrier(dist)
    wall_total = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    launches = model.launch_count() - launches0
    h2d1, d2h1 = model.transfer_bytes()

    wall_max = all_max(dist, wall_total)
    dev_max = all_max(dist, dev_ms / 1e3)
    tokens_all = all_sum(dist, float(tokens))
    generated_all = all_sum(dist, float(generated))
    pk = peaks()

    # one extra profiled step: CUDA events around every launch, per kernel class
    roof = None
    if (rank == 0 or ep) and not args.no_profiled_step:  # under expert parallelism every forward needs all ranks
        model.profile_enable(True)
        run_step(eng_mod, model, w, reqs, active, lockstep)
        prof_rows = model.profile_query()
        model.profile_enable(False)
        total_ms = sum(r["ms"] for r in prof_rows) or 1.0
        top = max(prof_rows, key=lambda r: r["ms"])
        intensity = top["flops"] / max(top["bytes"], 1.0)
        ridge = pk["tflops"] * 1e12 / (pk["hbm_gbs"] * 1e9)
        if top["flops"] > 0 and intensity > ridge:
            achieved = top["flops"] / (top["ms"] / 1e3) / 1e12
            roof = dict(bound="tensor", achieved=achieved, peak=pk["tflops"], unit="TFLOP/s", frac=achieved / pk["tflops"], traffic=None)
        else:
            achieved = top["bytes"] / (top["ms"] / 1e3) / 1e9
            roof = dict(bound="hbm", achieved=achieved, peak=pk["hbm_gbs"], unit="GB/s", frac=achieved / pk["hbm_gbs"], traffic=None)
        ratio = NCU_TRAFFIC_RATIO.get(top["name"])
        if ratio is not None:
            roof["traffic"] = ratio * top["bytes"] / max(top["launches"], 1)
            roof["traffic_unit"] = "bytes per launch (ncu ratio x live algorithmic bytes)"
        roof.update(kernel=top["name"], launches=top["launches"], avg_launch_ms=top["ms"] / max(top["launches"], 1),
                    time_share=top["ms"] / total_ms, peak_source=pk["source"],
                    classes={r["name"]: dict(launches=r["launches"], ms=round(r["ms"], 3), share=round(r["ms"] / total_ms, 4),
                                             gbs=round(r["bytes"] / max(r["ms"], 1e-9) / 1e6, 1),
                                             tflops=round(r["flops"] / max(r["ms"], 1e-9) / 1e9, 2)) for r in prof_rows})

    classes = None
    if (rank == 0 or ep) and not args.no_profiled_step:
        sliding = (spec.layers // 2, spec.layers, spec.window) if spec.arch == "gemma2" else (0, 0, 0)
        weights_pass = float(wb["per_token"]) if spec.experts == 0 else float(wb.get("all_experts", wb["per_token"]))
        if ep:  # this rank's share: everything but the expert banks, plus its experts
            expert_part = float(wb.get("experts_only", 0.0))
            weights_pass = weights_pass - expert_part + expert_part / world
        classes = tick_classes(eng_mod, model, w, reqs, active, weights_pass, float(model.spec().kv_bytes_per_token), pk["hbm_gbs"], sliding, lockstep)
        if roof is not None and "decode" in classes:
            # the decode roofline of the metric: weight + K/V bytes of a tick over its device time
            d = classes["decode"]
            roof["decode_tick"] = dict(achieved=d["gbs"], peak=pk["hbm_gbs"], unit="GB/s", frac=d["hbm_frac"], ms_per_tick=d["ms_per_tick"],
                                       lanes_per_tick=d["lanes_per_tick"])
        if roof is not None:
            roof["q4k_gemv"] = q4k_gemv_block(pk["hbm_gbs"])

    http = None
    if rank == 0 and args.http_clients > 0 and not ep:
        http = http_step(eng_mod, model, w, reqs, active, args.http_clients)

    base = None
    if rank == 0 and not args.no_cpu_baseline:
        try:
            base = cpu_baseline(w, path, 15.0, max(1, (os.cpu_count() or 1)))
        except Exception as e:  # the baseline is a report, never a reason to lose the measurement
            base = dict(value=None, unit=UNIT, cores=None, kind="port", sample=f"failed: {e}")

    # the headline line is complete before the sparse-MoE slice starts: whatever becomes of the slice, it is printed once
    out = None
    if rank == 0:
        out = dict(metric=METRIC, value=tokens_all / dev_max, unit=UNIT, n_gpus=world, steps=args.steps, warmup=args.warmup,
                   ms_per_step=wall_max * 1e3 / max(args.steps, 1), higher_is_better=True, scaling="weak", vs_baseline=None,
                   dtype="f16 tensor cores over f16 weights dequantised in flight (1..64 rows) or f16 weight images (wider ticks), f32 accumulate, f16 KV",
                   data="synthetic", config=config, clocks=clocks,
                   e2e=dict(value=tokens_all / wall_max, unit=UNIT, h2d_bytes_per_step=(h2d1 - h2d0) // max(args.steps, 1),
                            d2h_bytes_per_step=(d2h1 - d2h0) // max(args.steps, 1)),
                   gpu_launches=launches, ticks_per_step=ticks // max(args.steps, 1),
                   # the reference's scoreboard also quotes generated tokens alone (src/benchmark/serving.rs:301-328)
                   output_tokens_per_s=generated_all / dev_max, roofline=roof, tick_classes=classes,
                   cpu_baseline=base)
        out["forward_kinds_ms_per_step"] = {k: round(v / max(args.steps, 1), 3) for k, v in forward_kinds.items()}
        if diag is not None:
            out["prefix_cache"] = diag
        if http is not None:
            out["http"] = http
    emit = line_emitter(out)

    # the sparse-MoE curve beside the headline (every rank takes part; the headline model's memory is released first)
    ep_block = None
    if args.workload == DEFAULT_WORKLOAD and not sliced and not args.no_ep_slice and not args.no_profiled_step:
        model.close()
        # should the slice outlast its deadline (a rank stuck in a collective), rank 0 prints the headline without it
        timer = threading.Timer(EP_SLICE_DEADLINE_S, emit, kwargs=dict(ep=dict(error=f"the slice did not finish within {EP_SLICE_DEADLINE_S:.0f} s")))
        timer.daemon = True
        timer.start()
        try:
            ep_block = ep_slice(eng_mod, wl, seed, rank, local, world, dist, args.kv_budget_gb)
        except Exception as e:  # never a reason to lose the headline measurement
            ep_block = dict(error=str(e)[:400])
        timer.cancel()
    emit(ep=ep_block)
    model.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
