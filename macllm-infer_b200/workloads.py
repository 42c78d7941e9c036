"""The five benchmark workloads: model shape, engine settings and seeded synthetic requests.

No public suite or dataset is involved: token ids are uniform in [3, vocab) from a seeded generator, prompt lengths
follow the stated distributions, arrival times (workload 5) are a seeded Poisson process.  The engine settings follow the
reference's defaults where it has them (src/engine.rs:335-348: quantum 128, budget 256) and its prefix demo
(src/benchmark/prefix_demo_mac.rs:39-42: prefix capacity 65 536 tokens, budget 1 024).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class Workload:
    name: str
    config: str                   # key of seed_gguf.CONFIGS
    seqs: int                     # requests per replica
    new_tokens: int | tuple       # tokens per request, or (low, high) uniform
    quantum: int
    budget: int
    seed: int
    active: int = 0               # max_active_sequences (0 = seqs)
    prompt: tuple | None = None   # uniform (low, high)
    prompt_list: list | None = None
    lognormal: tuple | None = None       # (median, sigma, low, high)
    shared_prefix: int = 0               # tokens every request of the replica starts with
    prefix_capacity_tokens: int = 0
    arrival_rate: float = 0.0            # requests per second (Poisson); 0 = all at once as one atomic batch
    kv_slack: int = 32
    extra: dict = field(default_factory=dict)

    def max_active(self) -> int:
        return self.active or self.seqs


WORKLOADS = {
    # 1: 4 sequences 17/64/128/301, 32 tokens, the reference's default quantum and budget
    "tinyllama-1.1b-batch4": Workload("tinyllama-1.1b-batch4", "tinyllama-1.1b", 4, 32, 128, 256, 1001, prompt_list=[17, 64, 128, 301]),
    # 2: 64 sequences U[32, 1024], 512-token chunks, 128 tokens
    "smollm3-3b-ragged64": Workload("smollm3-3b-ragged64", "smollm3-3b", 64, 128, 512, 2048, 1002, prompt=(32, 1024)),
    # 3: per replica 32 requests = 2048 shared tokens + U[16, 256] suffix, 256 tokens, prefix cache on; request 0 runs
    #    alone first, then the rest in submission order
    "qwen3-8b-prefix32": Workload("qwen3-8b-prefix32", "qwen3-8b", 32, 256, 512, 1024, 1003, prompt=(16, 256), shared_prefix=2048,
                                  prefix_capacity_tokens=65536),
    # 4: 128 sequences, prompts lognormal (median 3000) clipped to [256, 8192], 256 tokens, sliding-window layers
    "gemma2-9b-long128": Workload("gemma2-9b-long128", "gemma2-9b", 128, 256, 512, 2048, 1004, lognormal=(3000.0, 0.6, 256, 8192)),
    # 5: Poisson arrivals at 64 requests/s for 60 s, prompts U[64, 2048], outputs U[64, 512], up to 512 concurrent
    "qwen3-30b-a3b-poisson": Workload("qwen3-30b-a3b-poisson", "qwen3-30b-a3b", 3840, (64, 512), 512, 4096, 1005, active=512,
                                      prompt=(64, 2048), arrival_rate=64.0),
}


def make_requests(w: Workload, vocab: int, rank: int = 0, limit: int = 0):
    """Returns (prompts, new_tokens per request, arrival time in seconds per request) for one replica."""
    rng = np.random.default_rng(w.seed + 7919 * rank)
    n = w.seqs if limit <= 0 else min(w.seqs, limit)
    if w.prompt_list is not None:
        lens = list(w.prompt_list)[:n]
    elif w.lognormal is not None:
        med, sigma, lo, hi = w.lognormal
        lens = [int(min(hi, max(lo, round(float(x))))) for x in rng.lognormal(np.log(med), sigma, size=w.seqs)][:n]
    else:
        lens = [int(x) for x in rng.integers(w.prompt[0], w.prompt[1] + 1, size=w.seqs)][:n]
    prefix = rng.integers(3, vocab, size=w.shared_prefix).astype(np.uint32) if w.shared_prefix else None
    prompts = []
    for k in lens:
        body = rng.integers(3, vocab, size=k).astype(np.uint32)
        prompts.append(np.concatenate([prefix, body]) if prefix is not None else body)
    if isinstance(w.new_tokens, tuple):
        new = [int(x) for x in rng.integers(w.new_tokens[0], w.new_tokens[1] + 1, size=w.seqs)][:n]
    else:
        new = [int(w.new_tokens)] * n
    if w.arrival_rate > 0:
        arrivals = list(np.cumsum(rng.exponential(1.0 / w.arrival_rate, size=w.seqs))[:n])
    else:
        arrivals = [0.0] * n
    return prompts, new, arrivals


def kv_capacity_tokens(w: Workload, prompts, new) -> int:
    """A pool that holds the whole active set at its longest (16-token blocks, one block of slack per sequence)."""
    longest = sorted((len(p) + k + w.kv_slack for p, k in zip(prompts, new)), reverse=True)
    return int(sum(longest[: w.max_active()])) + (w.prefix_capacity_tokens and 0)
