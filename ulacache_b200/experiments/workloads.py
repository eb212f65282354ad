"""Frozen, hash-pinned workloads for the serving and capacity experiments.

    python -m ulacache_b200.experiments.workloads prepare-documents OUT.jsonl.gz [--count 64] [--mean-tokens 98000]
    python -m ulacache_b200.experiments.workloads prepare-conversations OUT.jsonl.gz [--sessions 512] [--turns 4,12]
    python -m ulacache_b200.experiments.workloads verify OUT.jsonl.gz

The reference's studies run on two frozen datasets: long legal documents (Multi-LexSum, about 98 K tokens per
document on average) for the capacity / throughput studies, and multi-turn agent conversations with a shared system
prefix for the online-serving study.  The datasets themselves need the network; what the experiments depend on is
their SHAPE (length distribution, turn structure, prefix sharing) and that every method replays byte-identical
requests.  A workload file here is generated from a seed with those shapes, carries a manifest line with its
parameters and the SHA-256 of its payload, and is refused by the loader when the hash differs - so two runs (two
cache methods, two machines) are known to have served the same requests.  Token values are uniform random: nothing
in the cache depends on them.

Reference: scripts/datasets/prepare_multilexsum.py, scripts/datasets/prepare_rightfit.py (frozen, hash-pinned
long-context workloads); scripts/7_1_online/run.py (conversation replay).
"""
from __future__ import annotations

import argparse
import gzip
import hashlib
import json
import math
import random
from typing import Dict, Iterable, List, Optional

SCHEMA = "ulc-workload-v1"


def _payload_lines(records: Iterable[dict]) -> List[bytes]:
    return [json.dumps(r, sort_keys=True, separators=(",", ":")).encode() for r in records]


def write_workload(path: str, kind: str, params: dict, records: Iterable[dict]) -> str:
    """Manifest line + one JSON line per record, gzip with a zero timestamp (reproducible bytes).  Returns the payload hash."""
    lines = _payload_lines(records)
    digest = hashlib.sha256(b"\n".join(lines)).hexdigest()
    manifest = dict(schema=SCHEMA, kind=kind, params=params, records=len(lines), payload_sha256=digest)
    raw = b"\n".join([json.dumps(manifest, sort_keys=True).encode()] + lines) + b"\n"
    with open(path, "wb") as f:
        f.write(gzip.compress(raw, mtime=0) if path.endswith(".gz") else raw)
    return digest


def load_workload(path: str, expected_sha256: Optional[str] = None) -> Dict:
    """{"manifest": ..., "records": [...]}; ValueError when the payload does not hash to the manifest (or to
    ``expected_sha256``: what the other arm of a comparison served)."""
    with open(path, "rb") as f:
        raw = f.read()
    if raw[:2] == b"\x1f\x8b":
        raw = gzip.decompress(raw)
    head, _, body = raw.partition(b"\n")
    manifest = json.loads(head)
    if manifest.get("schema") != SCHEMA:
        raise ValueError("not a workload file of this schema")
    lines = [l for l in body.split(b"\n") if l]
    digest = hashlib.sha256(b"\n".join(lines)).hexdigest()
    if digest != manifest["payload_sha256"] or len(lines) != manifest["records"]:
        raise ValueError("workload payload differs from its manifest")
    if expected_sha256 is not None and digest != expected_sha256:
        raise ValueError("this is not the workload the other arm served")
    return dict(manifest=manifest, records=[json.loads(l) for l in lines])


def long_documents(*, count: int = 64, mean_tokens: int = 98000, sigma: float = 0.55, min_tokens: int = 8192,
                   max_tokens: int = 262144, vocab: int = 129280, output_tokens: int = 256, seed: int = 0) -> List[dict]:
    """Documents with log-normal lengths (mean ``mean_tokens``) as single-turn requests: summarise-the-document."""
    rng = random.Random(seed)
    mu = math.log(mean_tokens) - sigma * sigma / 2.0          # mean of a log-normal = exp(mu + sigma^2 / 2)
    out = []
    for i in range(count):
        n = int(min(max_tokens, max(min_tokens, rng.lognormvariate(mu, sigma))))
        out.append(dict(rid=i, session=i, turn=0, arrival=0.0, prompt_tokens=n, prompt_seed=rng.getrandbits(48),
                        max_new=output_tokens, vocab=vocab))
    return out


def conversations(*, sessions: int = 512, turns_lo: int = 4, turns_hi: int = 12, system_prefix: int = 4096,
                  median_input: int = 512, sigma: float = 0.8, input_cap: int = 8192, out_lo: int = 64, out_hi: int = 512,
                  rate: float = 4.0, vocab: int = 129280, seed: int = 0) -> List[dict]:
    """Multi-turn sessions over one shared system prefix; every turn's prompt is the whole history so far.  Prompts
    are stored as (seed, length) segments, expanded by :func:`expand_prompt`, so a file of thousands of long
    requests stays small."""
    rng = random.Random(seed)
    system_seed = rng.getrandbits(48)
    turns = [rng.randint(turns_lo, turns_hi) for _ in range(sessions)]
    history = [[(system_seed, system_prefix)] for _ in range(sessions)]
    t, rid, out = 0.0, 0, []
    for turn in range(max(turns)):
        for s in range(sessions):
            if turn >= turns[s]:
                continue
            t += rng.expovariate(rate)
            n_in = int(min(input_cap, max(1, rng.lognormvariate(math.log(median_input), sigma))))
            n_out = rng.randint(out_lo, out_hi)
            history[s] = history[s] + [(rng.getrandbits(48), n_in)]
            out.append(dict(rid=rid, session=s, turn=turn, arrival=round(t, 6), segments=[list(x) for x in history[s]],
                            prompt_tokens=sum(n for _, n in history[s]), max_new=n_out, vocab=vocab))
            history[s] = history[s] + [(rng.getrandbits(48), n_out)]     # the reply joins the history
            rid += 1
    return out


def expand_prompt(record: dict) -> List[int]:
    """Token ids of a record's prompt (deterministic in the record alone)."""
    vocab = record["vocab"]
    segs = record.get("segments") or [[record["prompt_seed"], record["prompt_tokens"]]]
    toks: List[int] = []
    for seed, n in segs:
        r = random.Random(seed)
        toks.extend(r.randrange(vocab) for _ in range(n))
    return toks


def as_trace(workload: Dict, *, vocab: Optional[int] = None, limit: Optional[int] = None, max_prompt: Optional[int] = None):
    """Requests in the form the serving replay takes: dicts with rid, session, arrival, prompt, max_new."""
    out = []
    for rec in workload["records"][:limit]:
        if vocab is not None and rec["vocab"] != vocab:
            rec = dict(rec, vocab=vocab)
        prompt = expand_prompt(rec)
        if max_prompt is not None:
            prompt = prompt[:max_prompt]
        out.append(dict(rid=rec["rid"], session=rec["session"], arrival=rec["arrival"], prompt=prompt, max_new=rec["max_new"]))
    return out


def summary(workload: Dict) -> dict:
    lens = sorted(r["prompt_tokens"] for r in workload["records"])
    n = len(lens)
    return dict(kind=workload["manifest"]["kind"], records=n, payload_sha256=workload["manifest"]["payload_sha256"],
                prompt_tokens_mean=round(sum(lens) / max(n, 1), 1), prompt_tokens_p50=lens[n // 2] if n else 0,
                prompt_tokens_max=lens[-1] if n else 0, sessions=len({r["session"] for r in workload["records"]}),
                total_prompt_tokens=sum(lens))


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    d = sub.add_parser("prepare-documents")
    d.add_argument("out")
    d.add_argument("--count", type=int, default=64)
    d.add_argument("--mean-tokens", type=int, default=98000)
    d.add_argument("--seed", type=int, default=0)
    c = sub.add_parser("prepare-conversations")
    c.add_argument("out")
    c.add_argument("--sessions", type=int, default=512)
    c.add_argument("--turns", default="4,12")
    c.add_argument("--system-prefix", type=int, default=4096)
    c.add_argument("--rate", type=float, default=4.0)
    c.add_argument("--seed", type=int, default=0)
    v = sub.add_parser("verify")
    v.add_argument("path")
    v.add_argument("--sha256", default=None)
    args = ap.parse_args(argv)
    if args.cmd == "prepare-documents":
        params = dict(count=args.count, mean_tokens=args.mean_tokens, seed=args.seed)
        digest = write_workload(args.out, "long_documents", params, long_documents(**params))
    elif args.cmd == "prepare-conversations":
        lo, hi = (int(x) for x in args.turns.split(","))
        params = dict(sessions=args.sessions, turns_lo=lo, turns_hi=hi, system_prefix=args.system_prefix, rate=args.rate,
                      seed=args.seed)
        digest = write_workload(args.out, "conversations", params, conversations(**params))
    else:
        print(json.dumps(summary(load_workload(args.path, args.sha256))))
        return 0
    print(json.dumps(dict(path=args.out, payload_sha256=digest)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
