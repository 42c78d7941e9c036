"""The multi-GPU form of the benchmark is N independent replicas (one process per GPU, no data-path collective):
this exercises its plumbing - rendezvous, per-rank request streams, barrier, sum of tokens over ranks, time of the
slowest rank - with two CPU processes over gloo, each running the real engine (scheduler, paged KV pool, prefix
cache) on the host-only fake model."""
import json
import os
import socket
import subprocess
import sys
import textwrap
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

CHILD = textwrap.dedent("""
    import importlib, json, sys, time
    sys.path.insert(0, %r)
    import bench
    import __graft_entry__ as entry
    entry.load_package()
    eng = importlib.import_module("macllm_infer_b200.engine")
    rank, local, world, dist = bench.dist_setup(2, backend="gloo")
    wl = bench.workloads_module()
    w = wl.Workload("gloo-test", "none", 6, 7, 16, 64, 77, prompt=(5, 40))
    reqs = wl.make_requests(w, 32, rank)
    prompts = reqs[0]
    model = eng.Model.fake(vocab=32, max_context=256, kv_capacity_tokens=1024)
    bench.barrier(dist)
    tokens, seconds, st, _ = bench.run_step(eng, model, w, reqs, 6)   # the benchmark's own step driver
    seconds += 0.01 * (rank + 1)   # rank 1 is the slowest by construction
    assert tokens == sum(len(p) for p in prompts) + 6 * 7 and st["completed_requests"] == 6
    bench.barrier(dist)
    total, slowest, rate = bench.aggregate(dist, tokens, seconds)
    print(json.dumps(dict(rank=rank, world=world, tokens=tokens, seconds=seconds, total=total, slowest=slowest, rate=rate,
                          first_prompt=[int(x) for x in prompts[0][:4]])), flush=True)
    dist.destroy_process_group()
""") % str(ROOT)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_replicas_aggregate_over_gloo():
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, "-c", CHILD], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        out, err = p.communicate(timeout=240)
        assert p.returncode == 0, err[-2000:]
        outs.append(json.loads(out.strip().splitlines()[-1]))
    outs.sort(key=lambda o: o["rank"])
    assert [o["world"] for o in outs] == [2, 2]
    # per-rank request streams differ, every rank reports the same whole-job figures
    assert outs[0]["first_prompt"] != outs[1]["first_prompt"]
    want_total = outs[0]["tokens"] + outs[1]["tokens"]
    want_slowest = max(outs[0]["seconds"], outs[1]["seconds"])
    for o in outs:
        assert o["total"] == want_total
        assert abs(o["slowest"] - want_slowest) < 1e-9
        assert abs(o["rate"] - want_total / want_slowest) < 1e-6 * o["rate"]
    assert outs[1]["seconds"] == want_slowest


LOCKSTEP_CHILD = textwrap.dedent("""
    import importlib, json, sys
    sys.path.insert(0, %r)
    import bench
    import __graft_entry__ as entry
    entry.load_package()
    eng = importlib.import_module("macllm_infer_b200.engine")
    rank, local, world, dist = bench.dist_setup(2, backend="gloo")
    wl = bench.workloads_module()
    # rank 0 has twice the requests of rank 1, and Poisson arrivals: the ranks run out of lanes at different ticks
    w = wl.Workload("lockstep-test", "none", 8 if rank == 0 else 4, (3, 9), 16, 64, 78, prompt=(5, 40), arrival_rate=200.0)
    reqs = wl.make_requests(w, 32, rank)

    class Counting:
        # the host-only model with the expert-parallel idle tick of a GGUF model stubbed: counts the ticks this rank idles
        def __init__(self, inner):
            self.inner, self.idle = inner, 0
        def ep_idle_tick(self):
            self.idle += 1
        def __getattr__(self, name):
            return getattr(self.inner, name)

    model = Counting(eng.Model.fake(vocab=32, max_context=256, kv_capacity_tokens=2048))
    calls = [0]
    agree = bench.make_lockstep(dist)
    def lockstep(n, failed=False):
        calls[0] += 1
        return agree(n, failed)
    e = bench.new_engine(eng, model.inner, w, 4, len(reqs[0]))
    lanes = [n for n in bench.drive(eng, model, e, w, reqs, lockstep)]
    done = [e.result(i)["state"] for i in bench.drive.last_ids]
    print(json.dumps(dict(rank=rank, iterations=len(lanes), forwards=sum(1 for n in lanes if n > 0), idle=model.idle, calls=calls[0],
                          done=done, generated=sum(len(e.result(i)["tokens"]) for i in bench.drive.last_ids), want=int(sum(reqs[1])))), flush=True)
    dist.destroy_process_group()
""") % str(ROOT)


def test_lock_step_drive_keeps_two_ranks_on_the_same_tick_count():
    """The host loop of expert parallelism with data-parallel lanes (bench.drive with a lock-step sum, the same loop as
    engine.run_expert_parallel): every rank ticks until no rank has work left, a rank whose scheduler ran no lane takes the
    tick idle, and every request still finishes with its own token count."""
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, "-c", LOCKSTEP_CHILD], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        out, err = p.communicate(timeout=240)
        assert p.returncode == 0, err[-2000:]
        outs.append(json.loads(out.strip().splitlines()[-1]))
    outs.sort(key=lambda o: o["rank"])
    a, b = outs
    assert a["iterations"] == b["iterations"] and a["calls"] == b["calls"] == a["iterations"] + 1
    for o in outs:
        assert o["forwards"] + o["idle"] == o["iterations"]          # exactly one forward or one idle tick per iteration
        assert set(o["done"]) == {"done"} and o["generated"] == o["want"]
    assert b["idle"] > 0 and b["forwards"] < a["forwards"] + a["idle"]  # the rank with fewer requests idled through the tail


FAILURE_CHILD = textwrap.dedent("""
    import importlib, json, sys
    sys.path.insert(0, %r)
    import bench
    import __graft_entry__ as entry
    entry.load_package()
    eng = importlib.import_module("macllm_infer_b200.engine")
    rank, local, world, dist = bench.dist_setup(2, backend="gloo")
    wl = bench.workloads_module()
    w = wl.Workload("lockstep-failure", "none", 6, 8, 16, 64, 79, prompt=(5, 40))
    reqs = wl.make_requests(w, 32, rank)

    class Idle:
        def __init__(self, inner):
            self.inner = inner
        def ep_idle_tick(self):
            pass
        def __getattr__(self, name):
            return getattr(self.inner, name)

    inner = eng.Model.fake(vocab=32, max_context=256, kv_capacity_tokens=2048)
    if rank == 1:
        inner.inject_failure("forward", 3)      # rank 1's fourth forward fails: its engine poisons, its requests fail
    outcome = "ok"
    try:
        bench.run_step(eng, Idle(inner), w, reqs, 6, bench.make_lockstep(dist))
    except RuntimeError as e:
        outcome = str(e)
    print(json.dumps(dict(rank=rank, outcome=outcome)), flush=True)
    dist.barrier()          # both ranks are still in step: nobody was left inside a collective
    dist.destroy_process_group()
""") % str(ROOT)


def test_a_failure_on_one_rank_ends_the_lock_step_on_all_of_them():
    """One rank's model fails mid-run: that rank's requests end failed, it keeps ticking idle until the group is done, and
    the agreement at the end of the step makes BOTH ranks raise - the healthy one with a message naming a peer - instead of
    one of them waiting in a collective for ever."""
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, "-c", FAILURE_CHILD], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        out, err = p.communicate(timeout=120)
        assert p.returncode == 0, err[-2000:]
        outs.append(json.loads(out.strip().splitlines()[-1]))
    outs.sort(key=lambda o: o["rank"])
    assert "another rank" in outs[0]["outcome"]
    assert "ended in state failed" in outs[1]["outcome"] and "inference worker failed" in outs[1]["outcome"]


def test_the_headline_line_is_printed_once_whatever_becomes_of_the_slice(capsys):
    """bench.line_emitter: the headline is complete before the sparse-MoE slice starts; the first of (slice finished, slice
    overdue) prints it, the other does nothing; ranks that print nothing still take part."""
    import threading
    import time
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench
    emit = bench.line_emitter(dict(metric="m", value=1.0))
    overdue = threading.Timer(0.05, emit, kwargs=dict(ep=dict(error="the slice did not finish")))
    overdue.start()
    time.sleep(0.3)
    assert emit(ep=dict(value=2.0)) is False
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 1 and json.loads(lines[0]) == {"metric": "m", "value": 1.0, "ep": {"error": "the slice did not finish"}}
    emit = bench.line_emitter(dict(metric="m", value=1.0))
    waiting = threading.Timer(30.0, emit)
    waiting.daemon = True
    waiting.start()
    waiting.cancel()
    assert emit(ep=dict(value=2.0)) is True and emit() is False
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 1 and json.loads(lines[0])["ep"] == {"value": 2.0}
    silent = bench.line_emitter(None)
    assert silent(ep=1) is True and capsys.readouterr().out == ""
