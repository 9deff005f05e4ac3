"""Synthetic batch workloads of the benchmark configurations, as OpenAI-style batch JSONL files.

Every profile is defined by prompt lengths, decode lengths and how prompts share prefixes; token ids are
uniform random (seeded), completions are forced to their full length (``ignore_eos``).  ``--scale`` shrinks
lengths and counts proportionally so that the same shape runs on a small model or a CPU.

  tiny            8 requests x 32 tokens, 16 decode tokens                         (correctness config)
  mixed-1k        512 requests, prompts U[512, 4096], 1,024 decode tokens          (DeepSeek-V3/R1 config)
  long-distinct   312 distinct 65,536-token prompts, 4,096 decode tokens           (GLM-5.3 sparse prefill)
  long-grouped    64 prefixes of 65,536 tokens x 8 suffixes of 64, 4,096 decode    (prefix reuse)
  short-long      512 requests, prompts U[200, 1500], 4,096 decode tokens          (Kimi-K3 long decode)

Reference parity: benchmarks/decode_workload.py + configs/decode_workloads.json (workload profiles),
benchmarks/README.md:7-18 (batch completion time = first request issued to last completion received).
"""
from __future__ import annotations

import argparse
import json
import random
import sys
from dataclasses import dataclass
from typing import Iterator, List, Optional, Tuple


@dataclass(frozen=True)
class Profile:
    name: str
    requests: int
    prompt_range: Tuple[int, int]
    decode_tokens: int
    groups: int = 0                  # > 0: that many shared prefixes, requests / groups members each
    suffix_tokens: int = 0


PROFILES = {p.name: p for p in (
    Profile("tiny", 8, (32, 32), 16),
    Profile("mixed-1k", 512, (512, 4096), 1024),
    Profile("long-distinct", 312, (65536, 65536), 4096),
    Profile("long-grouped", 512, (65536, 65536), 4096, groups=64, suffix_tokens=64),
    Profile("short-long", 512, (200, 1500), 4096),
)}


def scaled(p: Profile, scale: float) -> Profile:
    if scale == 1.0:
        return p
    f = lambda v, lo=1: max(lo, int(round(v * scale)))
    groups = max(1, f(p.groups)) if p.groups else 0
    reqs = f(p.requests, 2)
    if groups:
        reqs = max(groups, reqs // groups * groups)
    return Profile(p.name, reqs, (f(p.prompt_range[0], 4), f(p.prompt_range[1], 4)), f(p.decode_tokens, 2), groups,
                   f(p.suffix_tokens, 2) if p.suffix_tokens else 0)


def prompts(p: Profile, vocab: int, seed: int = 0) -> Iterator[List[int]]:
    rng = random.Random(seed)
    tok = lambda: rng.randrange(2, vocab)
    if p.groups:
        per = p.requests // p.groups
        for _ in range(p.groups):
            prefix = [tok() for _ in range(rng.randint(*p.prompt_range))]
            for _ in range(per):
                yield prefix + [tok() for _ in range(p.suffix_tokens)]
    else:
        for _ in range(p.requests):
            yield [tok() for _ in range(rng.randint(*p.prompt_range))]


def batch_lines(p: Profile, vocab: int, seed: int = 0, model: str = "model") -> Iterator[str]:
    for i, ids in enumerate(prompts(p, vocab, seed)):
        yield json.dumps({"custom_id": f"{p.name}-{i}", "method": "POST", "url": "/v1/completions",
                          "body": {"model": model, "prompt": ids, "max_tokens": p.decode_tokens, "temperature": 0,
                                   "ignore_eos": True}})


def summary(p: Profile) -> dict:
    lo, hi = p.prompt_range
    mean_prompt = (lo + hi) / 2 + p.suffix_tokens
    return {"profile": p.name, "requests": p.requests, "mean_prompt_tokens": mean_prompt,
            "prompt_tokens_total": int(mean_prompt * p.requests), "decode_tokens_total": p.decode_tokens * p.requests,
            "shared_prefix_groups": p.groups}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="write a synthetic batch workload as JSONL")
    ap.add_argument("profile", choices=sorted(PROFILES))
    ap.add_argument("--out", required=True)
    ap.add_argument("--vocab", type=int, default=129280)
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    p = scaled(PROFILES[a.profile], a.scale)
    with open(a.out, "w") as f:
        for line in batch_lines(p, a.vocab, a.seed):
            f.write(line + "\n")
    print(json.dumps(summary(p)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
