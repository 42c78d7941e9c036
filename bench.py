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

N > 1 (torchrun) runs N independent replicas, one per GPU, each with its own request stream (the path
has no exchange step for dense models); the reported time is the max over ranks.
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

WORKLOADS = {
    # name: (seed config, sequences, prompt range, new tokens, quantum, budget)
    "smollm3-3b-ragged64": dict(config="smollm3-3b", seqs=64, prompt=(32, 1024), new_tokens=128, quantum=512, budget=2048, seed=1002),
    "tinyllama-1.1b-batch4": dict(config="tinyllama-1.1b", seqs=4, prompt_list=[17, 64, 128, 301], new_tokens=32, quantum=128,
                                  budget=256, seed=1001),
}


# DRAM traffic of the three dominant kernels relative to their algorithmic bytes, from one `ncu --set full` capture
# each on the benchmark's shapes (dram__bytes_read.sum + dram__bytes_write.sum over the bytes counted here).  The
# roofline block scales the live per-launch algorithmic bytes by these ratios.
NCU_TRAFFIC_RATIO = {
    "hgemm_tc": (98.8 + 21.4) / (90.2 + 8.4 + 45.1),      # gate|up with the activation in the epilogue: every operand once; part of the f16 output is still in L2 at kernel end
    "qstream_tc": 25.69 / (25.36 + 0.26 + 5.64),          # weights once; the partial sums never leave L2
    "paged_attention": (77.0 + 1.9) / (72.4 + 4.2),
}


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback")


def make_prompts(w: dict, vocab: int, rank: int):
    rng = np.random.default_rng(w["seed"] + 7919 * rank)
    if "prompt_list" in w:
        lens = list(w["prompt_list"])
    else:
        lens = [int(x) for x in rng.integers(w["prompt"][0], w["prompt"][1] + 1, size=w["seqs"])]
    return [rng.integers(3, vocab, size=n).astype(np.uint32) for n in lens]


def checkpoint_path(w: dict) -> Path:
    d = Path(os.environ.get("MACLLM_SEED_DIR", tempfile.gettempdir())) / "macllm_b200_seed"
    d.mkdir(parents=True, exist_ok=True)
    return d / f"{w['config']}.gguf"


def ensure_checkpoint(w: dict) -> Path:
    seed = importlib.import_module("macllm_infer_b200.seed_gguf")
    path = checkpoint_path(w)
    done = path.with_suffix(".done")
    if not done.exists():
        t0 = time.time()
        seed.write_seed_gguf(path, seed.CONFIGS[w["config"]], seed=0)
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


def run_step(eng_mod, model, w, prompts):
    """One step: the whole continuous batch through a fresh engine.  Returns (tokens, wall s, stats)."""
    eng = eng_mod.Engine(model, max_active_sequences=w["seqs"], scheduler_token_budget=w["budget"],
                         prefill_token_quantum=w["quantum"], queue_capacity=w["seqs"] + 8)
    reqs = [eng_mod.Request(p, w["new_tokens"]) for p in prompts]
    model.synchronize()
    t0 = time.perf_counter()
    ids = eng.submit(reqs, atomic_batch=True)
    eng.run()
    model.synchronize()
    wall = time.perf_counter() - t0
    st = eng.stats()
    toks = sum(len(p) for p in prompts)
    gen = 0
    for i in ids:
        r = eng.result(i)
        if r["state"] != "done":
            raise RuntimeError(f"request {i} ended in state {r['state']}: {r['message']}")
        gen += len(r["tokens"])
    eng.close()
    return toks + gen, wall, st


def tick_classes(eng_mod, model, w, prompts, weight_bytes_per_pass: float, kv_bytes_per_token: float, hbm_gbs: float) -> dict:
    """One more (untimed) step driven tick by tick: device time and algorithmic HBM bytes per tick class.
    A tick's algorithmic bytes = the weight bytes one pass touches + the K/V history its lanes attend to;
    `hbm_frac` = those bytes / device time / measured copy bandwidth (the decode roofline of the metric)."""
    eng = eng_mod.Engine(model, max_active_sequences=w["seqs"], scheduler_token_budget=w["budget"],
                         prefill_token_quantum=w["quantum"], queue_capacity=w["seqs"] + 8)
    eng.submit([eng_mod.Request(p, w["new_tokens"]) for p in prompts], atomic_batch=True)
    ms = []
    while eng.pending() > 0:
        before = model.launch_count()
        eng.step()
        if model.launch_count() != before:  # a step that only delivers events runs no forward pass
            ms.append(model.last_forward_ms())
    trace = eng.trace()
    eng.close()
    out = {}
    for t, dev_ms in zip(trace, ms):
        toks = sum(n for _, _, n in t)
        if toks == 0:
            continue
        cls = "decode" if toks == len(t) else ("mixed" if any(n == 1 for _, _, n in t) else "prefill")
        kv = sum(sp + n for _, sp, n in t) * kv_bytes_per_token
        a = out.setdefault(cls, dict(ticks=0, tokens=0, ms=0.0, bytes=0.0))
        a["ticks"] += 1
        a["tokens"] += toks
        a["ms"] += dev_ms
        a["bytes"] += weight_bytes_per_pass + kv
    for a in out.values():
        a["tokens_per_s"] = round(a["tokens"] / max(a["ms"], 1e-9) * 1e3, 1)
        a["ms_per_tick"] = round(a["ms"] / a["ticks"], 3)
        a["hbm_frac"] = round(a["bytes"] / max(a["ms"], 1e-9) / 1e6 / hbm_gbs, 4)
        a["ms"] = round(a["ms"], 2)
        del a["bytes"]
    return out


Q4K_SHAPES = [(2048, 2048), (256, 2048), (5632, 2048), (2048, 5632), (11008, 2048), (2048, 11008), (12288, 4096)]


def microbench() -> None:
    """Q4_K matmul micro-benchmark: achieved GB/s on the algorithmic bytes of the matrix (rows * cols * 144/256) for
    the decode shapes of the first three configurations at 1, 4, 16 and 64 activation rows, on the path the model
    picks for that many rows (integer GEMV up to 8 rows, streamed blocks above).  Operands resident, L2 flushed
    before every launch, CUDA events around the launch.  One JSON line per shape."""
    ops = importlib.import_module("macllm_infer_b200.ops")
    capi = importlib.import_module("macllm_infer_b200._capi")
    pk = peaks()
    rng = np.random.default_rng(0)
    for rows, cols in Q4K_SHAPES:
        wq = ops.seed_tensor(0, 1, 0.02, capi.TYPE_Q4_K, rows, cols)
        nbytes = rows * cols * 144 // 256
        line = dict(kernel="q4k_matmul", rows=rows, cols=cols, weight_mb=round(nbytes / 1e6, 2), peak_gbs=pk["hbm_gbs"], peak_source=pk["source"])
        for T in (1, 4, 16, 64):
            x = rng.standard_normal((T, cols)).astype(np.float32)
            path = capi.PATH_GEMV if T <= 8 else capi.PATH_STREAM
            ms = ops.qmatmul_time(capi.TYPE_Q4_K, wq, rows, cols, x, path, 20)
            line[f"T{T}"] = dict(us=round(ms * 1e3, 1), gbs=round(nbytes / ms / 1e6, 1), frac=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
        print(json.dumps(line), flush=True)


def cpu_baseline(w, path, budget_s: float, seqs_sample: int = 4) -> dict:
    """The oracle (a port of the reference's CPU path) on a bounded sample of the same workload: the
    first prefill tokens of the first sequences, one scheduler tick, all host threads."""
    from oracle import decoder, engine as oe, mathlib
    mathlib.build()
    t0 = time.time()
    dec = decoder.Decoder(path, kv_dtype="f32", matmul_mode=1)
    load_s = time.time() - t0
    prompts = make_prompts(w, dec.vocab, 0)
    # calibrate on a short tick, then size the sample to the time budget
    def tick(n_tokens: int) -> float:
        om = oe.OracleModel(dec.vocab, dec.max_context, 16, 8, max(n_tokens + 64, 1024), 0, decoder=dec)
        s = om.new_session()
        ids = [int(x) for x in np.concatenate(prompts)[:n_tokens]]
        r = om.reserve_batch([(s, 0, len(ids))])
        t = time.time()
        om.forward([(s, ids, 0)], r)
        return time.time() - t
    probe = tick(8)
    n = int(max(8, min(512, budget_s / max(probe / 8, 1e-6))))
    dt = tick(n)
    return dict(value=n / dt, unit=UNIT, cores=mathlib.num_threads(), kind="port",
                sample=f"one prefill tick of {n} tokens of sequence 0 ({dt:.1f}s; checkpoint load {load_s:.1f}s not counted)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="smollm3-3b-ragged64", choices=list(WORKLOADS))
    ap.add_argument("--matmul-path", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    # a shorter slice of the same workload for profiler captures (a number printed by such a run is not a bench value)
    ap.add_argument("--new-tokens", type=int, default=0, help="override the generated tokens per sequence")
    ap.add_argument("--no-profiled-step", action="store_true", help="skip the extra step that times every launch")
    ap.add_argument("--microbench", action="store_true", help="Q4_K matmul GB/s on the decode shapes instead of the workload")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.new_tokens > 0:
        w["new_tokens"] = args.new_tokens

    rank, local, world, dist = dist_setup(args.gpus)
    entry.load_package()
    if rank == 0:
        entry.ensure_built()
    barrier(dist)
    seed = importlib.import_module("macllm_infer_b200.seed_gguf")
    spec = seed.CONFIGS[w["config"]]
    config = dict(workload=args.workload + (f" (slice: {w['new_tokens']} new tokens)" if args.new_tokens > 0 else ""), model_shape=w["config"], sequences_per_gpu=w["seqs"], new_tokens=w["new_tokens"],
                  prefill_quantum=w["quantum"], scheduler_token_budget=w["budget"], kv="f16 paged, 16-token blocks",
                  quant="Q4_K_M-shaped GGUF (Q4_K, Q6_K for attn_v and output)", parallelism=f"replicas x{world}",
                  l2="inputs larger than L2 (weights %.2f GB per pass)" % (seed.weight_bytes(spec)["per_token"] / 1e9))

    if args.microbench:
        if rank == 0:
            microbench()
        return

    if args.impl == "reference":
        # The reference is Rust on candle and cannot be built here (no cargo/rustc): the reference arm
        # is the CPU oracle, the port of its CPU path, on a bounded sample per step.
        if rank != 0:
            return
        path = ensure_checkpoint(w)
        budget = max(4.0, 150.0 / max(args.steps + args.warmup, 1))
        vals = []
        for i in range(args.warmup + args.steps):
            b = cpu_baseline(w, path, budget)
            if i >= args.warmup:
                vals.append(b)
        v = float(np.mean([b["value"] for b in vals])) if vals else 0.0
        b = vals[-1] if vals else dict(cores=0, sample="none", kind="port")
        out = dict(metric=METRIC, value=v, unit=UNIT, n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                   ms_per_step=None, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="int8 x int4/6 block dots, f32 accumulate",
                   data="synthetic", config=config, impl="reference",
                   cpu_baseline=dict(value=v, unit=UNIT, cores=b["cores"], kind=b["kind"], sample=b["sample"]),
                   e2e=dict(value=v, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
        print(json.dumps(out))
        return

    capi = importlib.import_module("macllm_infer_b200._capi")
    eng_mod = importlib.import_module("macllm_infer_b200.engine")
    if capi.lib().mk_device_count() <= 0:
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    if rank == 0:
        path = ensure_checkpoint(w)
    barrier(dist)
    path = checkpoint_path(w)

    prompts = make_prompts(w, spec.vocab, rank)
    max_len = max(len(p) for p in prompts) + w["new_tokens"]
    model = eng_mod.Model.load_gguf(path, device=local, kv_capacity_tokens=w["seqs"] * ((max_len + 15) // 16 * 16 + 16), kv_dtype="f16",
                                    max_batch_tokens=w["budget"], max_batch_lanes=w["seqs"], matmul_path=args.matmul_path)
    for _ in range(args.warmup):
        run_step(eng_mod, model, w, prompts)
    sampler = ClockSampler(local)
    barrier(dist)
    if rank == 0:
        sampler.start()
    launches0 = model.launch_count()
    h2d0, d2h0 = model.transfer_bytes()
    tokens = 0
    dev_ms = 0.0
    ticks = 0
    t0 = time.perf_counter()
    for _ in range(args.steps):
        n, wall, st = run_step(eng_mod, model, w, prompts)
        tokens += n
        dev_ms += st["device_ms"]
        ticks += st["ticks"]
    barrier(dist)
    wall_total = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    launches = model.launch_count() - launches0
    h2d1, d2h1 = model.transfer_bytes()

    wall_max = all_max(dist, wall_total)
    dev_max = all_max(dist, dev_ms / 1e3)
    tokens_all = all_sum(dist, float(tokens))

    # one extra profiled step: CUDA events around every launch, per kernel class
    roof = None
    prof_rows = []
    if rank == 0 and not args.no_profiled_step:
        model.profile_enable(True)
        run_step(eng_mod, model, w, prompts)
        prof_rows = model.profile_query()
        model.profile_enable(False)
        pk = peaks()
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
    if rank == 0 and not args.no_profiled_step:
        wb = seed.weight_bytes(spec)
        classes = tick_classes(eng_mod, model, w, prompts, float(wb["per_token"]), float(model.spec().kv_bytes_per_token),
                               peaks()["hbm_gbs"])

    base = None
    if rank == 0 and not args.no_cpu_baseline:
        try:
            base = cpu_baseline(w, path, 15.0)
        except Exception as e:  # the baseline is a report, never a reason to lose the measurement
            base = dict(value=None, unit=UNIT, cores=None, kind="port", sample=f"failed: {e}")

    if rank == 0:
        out = dict(metric=METRIC, value=tokens_all / dev_max, unit=UNIT, n_gpus=world, steps=args.steps, warmup=args.warmup,
                   ms_per_step=wall_max * 1e3 / max(args.steps, 1), higher_is_better=True, scaling="weak", vs_baseline=None,
                   dtype="f16 tensor cores over exact Q4_K integers or f16 weight images (>= 9 rows), int8 x int4/6 block dots (<= 8 rows), f32 accumulate, f16 KV",
                   data="synthetic", config=config, clocks=clocks,
                   e2e=dict(value=tokens_all / wall_max, unit=UNIT, h2d_bytes_per_step=(h2d1 - h2d0) // max(args.steps, 1),
                            d2h_bytes_per_step=(d2h1 - d2h0) // max(args.steps, 1)),
                   gpu_launches=launches, ticks_per_step=ticks // max(args.steps, 1), roofline=roof, tick_classes=classes,
                   cpu_baseline=base)
        print(json.dumps(out))
    model.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
