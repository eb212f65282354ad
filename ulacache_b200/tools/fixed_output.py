"""Replay samplers that make runs of different cache methods comparable: every method decodes
exactly the same token trajectory, so throughput differences come from the cache alone.

* :class:`FixedTokenReplay` - the "sampler" returns recorded tokens instead of model samples.
* :class:`FixedMTPReplay` - for speculative decoding: the number of accepted draft tokens per step
  is recorded too, so the verify batch sizes replay exactly.

Reference: ulacache/tools/fixed_output.py:60 (FixedMTPReplay), :243 (FixedTokenReplay).
"""
from __future__ import annotations

import json
from typing import Dict, List, Sequence


class ReplayExhausted(RuntimeError):
    pass


class FixedTokenReplay:
    def __init__(self, trajectories: Dict[int, Sequence[int]]):
        self.trajectories = {int(r): list(t) for r, t in trajectories.items()}
        self.cursor = {r: 0 for r in self.trajectories}

    @classmethod
    def record(cls, request_ids: Sequence[int], steps_of_tokens: Sequence[Sequence[int]]):
        """``steps_of_tokens[s][i]`` = token sampled for ``request_ids[i]`` at step s."""
        return cls({r: [step[i] for step in steps_of_tokens] for i, r in enumerate(request_ids)})

    def next_tokens(self, request_ids: Sequence[int]) -> List[int]:
        out = []
        for r in request_ids:
            c = self.cursor[r]
            if c >= len(self.trajectories[r]):
                raise ReplayExhausted(f"request {r} has no recorded token for step {c}")
            out.append(self.trajectories[r][c])
            self.cursor[r] = c + 1
        return out

    def remaining(self, request_id: int) -> int:
        return len(self.trajectories[request_id]) - self.cursor[request_id]

    def save(self, path: str):
        with open(path, "w") as f:
            json.dump({"kind": "fixed_tokens", "trajectories": self.trajectories}, f)

    @classmethod
    def load(cls, path: str):
        with open(path) as f:
            d = json.load(f)
        if d.get("kind") != "fixed_tokens":
            raise ValueError("not a fixed-token replay file")
        return cls({int(k): v for k, v in d["trajectories"].items()})


class FixedMTPReplay(FixedTokenReplay):
    """``accepts[r][s]`` = draft tokens accepted at verify step s (0..draft_steps); the step then
    emits ``accepts + 1`` tokens of the trajectory."""

    def __init__(self, trajectories, accepts: Dict[int, Sequence[int]], draft_steps: int):
        super().__init__(trajectories)
        self.accepts = {int(r): list(a) for r, a in accepts.items()}
        self.draft_steps = draft_steps
        self.step = {r: 0 for r in self.trajectories}
        for r, a in self.accepts.items():
            if any(x < 0 or x > draft_steps for x in a):
                raise ValueError("accepted length outside 0..draft_steps")
            if sum(x + 1 for x in a) > len(self.trajectories[r]):
                raise ValueError(f"request {r}: accepted lengths emit more tokens than were recorded")

    def next_verify(self, request_id: int) -> List[int]:
        s = self.step[request_id]
        if s >= len(self.accepts[request_id]):
            raise ReplayExhausted(f"request {request_id} has no recorded verify step {s}")
        n = self.accepts[request_id][s] + 1
        self.step[request_id] = s + 1
        return [self.next_tokens([request_id])[0] for _ in range(n)]


# ----------------------------------------------------------------------------------------------
# Recorded workloads: a trace file holds, per (attention-DP degree, repeat, batch, rank) case, the
# request order, the sequence positions and the tokens every step must emit.  A replay checks at
# every step that the engine presents the same requests at the same positions (otherwise the
# cache would be serving a different workload than the one recorded) and hands back the recorded
# tokens as tensors uploaded ONCE per cohort, so a measured step only selects a view.  A receipt
# states what was replayed and that no natural accuracy is claimed.
#
# Reference: ulacache/tools/fixed_output.py:13-57 (ReplayTrace), :60-241 (FixedMTPReplay with
# cohorts, frames and receipts), :243-346 (FixedTokenReplay begin / sample / end), :349-378
# (logits processor that forces the recorded token).
# ----------------------------------------------------------------------------------------------
import gzip
import hashlib

TOKEN_SCHEMA = "ulc-fixed-output-replay-v1"
MTP_SCHEMA = "ulc-fixed-mtp-replay-v1"


class ReplayMismatch(ValueError):
    pass


class ReplayTrace:
    """``data`` = {schema, output_tokens, speculative, cases: {"dp:repeat:batch:rank": episode name},
    episodes: {name: {...}}}.  Plain episodes: keys, input_tokens, saved_bootstrap_tokens,
    expected_output_ids {key: [tokens]}.  Speculative episodes: steps, verify_width, batch and
    frames [{keys, seq_lens, draft_tokens [[..]], accept_lens [..], emitted [[..]]}]."""

    def __init__(self, data: dict, raw: bytes = b""):
        self.data = data
        self.sha256 = hashlib.sha256(raw or json.dumps(data, sort_keys=True).encode()).hexdigest()
        schema = data.get("schema")
        self.speculative = schema == MTP_SCHEMA
        if self.speculative:
            if data.get("forced_acceptance") is not True:
                raise ValueError("a speculative replay trace must declare its forced acceptance")
        elif schema != TOKEN_SCHEMA or data.get("speculative") is not False:
            raise ValueError("not a recorded-output or speculative replay trace")
        budget = data["output_tokens"]
        for name, ep in data["episodes"].items():
            if self.speculative:
                if ep["verify_width"] != ep["steps"] + 1:
                    raise ValueError(f"episode {name}: a linear draft of n steps verifies n + 1 tokens")
                for f in ep["frames"]:
                    if any(not 1 <= a <= ep["verify_width"] for a in f["accept_lens"]):
                        raise ValueError(f"episode {name}: accepted length outside 1..verify width")
                    if any(len(e) != a for e, a in zip(f["emitted"], f["accept_lens"])):
                        raise ValueError(f"episode {name}: emitted tokens disagree with accepted lengths")
            elif any(len(ids) != budget for ids in ep["expected_output_ids"].values()):
                raise ValueError(f"episode {name}: recorded ids do not cover the output budget")

    @classmethod
    def load(cls, path: str):
        with open(path, "rb") as f:
            raw = f.read()
        text = gzip.decompress(raw) if raw[:2] == b"\x1f\x8b" else raw
        return cls(json.loads(text), raw)

    def save(self, path: str, compress: bool = True):
        text = json.dumps(self.data, sort_keys=True).encode()
        # mtime=0 keeps the bytes (and so the hash a client and a server compare) reproducible
        raw = gzip.compress(text, mtime=0) if compress else text
        with open(path, "wb") as f:
            f.write(raw)
        self.sha256 = hashlib.sha256(raw).hexdigest()
        return self.sha256

    def episode(self, attention_dp: int, repeat: int, batch: int, rank: int) -> dict:
        key = f"{attention_dp}:{repeat}:{batch}:{rank}"
        try:
            return self.data["episodes"][self.data["cases"][key]]
        except KeyError as err:
            raise ReplayMismatch(f"no recorded replay for case {key}") from err

    @classmethod
    def from_token_run(cls, *, attention_dp: int, repeat: int, rank: int, keys, input_tokens, outputs,
                       saved_bootstrap_tokens: int = 0):
        """Build a plain trace from one run: ``outputs[key]`` = every token the request emitted."""
        keys = list(keys)
        budget = len(outputs[keys[0]])
        ep = dict(keys=keys, input_tokens=list(input_tokens), saved_bootstrap_tokens=saved_bootstrap_tokens,
                  expected_output_ids={k: list(outputs[k]) for k in keys})
        return cls(dict(schema=TOKEN_SCHEMA, speculative=False, output_tokens=budget,
                        cases={f"{attention_dp}:{repeat}:{len(keys)}:{rank}": "e0"}, episodes={"e0": ep}))


class TraceTokenReplay:
    """Non-speculative replay of a recorded cohort: ``begin`` before the forward, ``sample`` in place of
    the sampler's result, ``end`` after the step."""

    def __init__(self, trace: ReplayTrace, *, attention_dp: int, rank: int):
        if trace.speculative:
            raise ValueError("a plain replay cannot use a speculative trace")
        self.trace, self.attention_dp, self.rank = trace, attention_dp, rank
        self.cohorts, self.active = {}, None

    def begin(self, cohort, *, repeat: int, keys, seq_lens, trace_sha256=None):
        if self.active is not None:
            raise ReplayMismatch("overlapping replay batches are not supported")
        if trace_sha256 is not None and trace_sha256 != self.trace.sha256:
            raise ReplayMismatch("client and server replay traces differ")
        st = self.cohorts.get(cohort)
        if st is None:
            ep = self.trace.episode(self.attention_dp, repeat, len(keys), self.rank)
            st = dict(episode=ep, position=ep["saved_bootstrap_tokens"], repeat=repeat, batch=len(keys), tensors=None,
                      forward_calls=0, sampler_calls=0)
            self.cohorts[cohort] = st
        ep, pos = st["episode"], st["position"]
        # input_tokens counts the prompt; the engine has appended every earlier output token to the sequence
        expected = [n + pos for n in ep["input_tokens"]]
        if list(keys) != ep["keys"] or list(seq_lens) != expected or pos >= self.trace.data["output_tokens"]:
            raise ReplayMismatch("replay request order or sequence positions differ from the recording")
        st["forward_calls"] += 1
        self.active = [cohort, st, False]

    def sample(self, natural):
        """``natural``: the sampler's own int tensor [batch]; returns the recorded tokens as a view of a tensor
        uploaded once per cohort (same shape, dtype and device)."""
        import torch

        if self.active is None:
            return natural
        cohort, st, sampled = self.active
        ep = st["episode"]
        if sampled or natural.ndim != 1 or natural.numel() != len(ep["keys"]) or natural.dtype not in (torch.int32, torch.int64):
            raise ReplayMismatch("a replay step takes exactly one greedy sampler call of the recorded batch")
        if st["tensors"] is None:
            st["tensors"] = torch.tensor([ep["expected_output_ids"][k] for k in ep["keys"]], dtype=natural.dtype,
                                         device=natural.device).T.contiguous()
        tokens = st["tensors"][st["position"]]
        st["position"] += 1
        st["sampler_calls"] += 1
        self.active[2] = True
        return tokens

    def end(self):
        if self.active is None or not self.active[2]:
            raise ReplayMismatch("the replay batch finished without its sampler call")
        self.active = None

    def completed(self, cohort) -> bool:
        return self.cohorts[cohort]["position"] == self.trace.data["output_tokens"]

    def receipt(self, cohort) -> dict:
        st = self.cohorts[cohort]
        return dict(trace_sha256=self.trace.sha256, attention_dp=self.attention_dp, rank=self.rank, repeat=st["repeat"],
                    batch=st["batch"], frames=st["sampler_calls"],
                    expected_frames=self.trace.data["output_tokens"] - st["episode"]["saved_bootstrap_tokens"],
                    forward_calls=st["forward_calls"], sampler_calls=st["sampler_calls"],
                    complete=self.completed(cohort), forced_acceptance=False, natural_accuracy_claimed=False)


class TraceMTPReplay:
    """Speculative replay: ``draft`` hands the verify pass its scripted draft tokens, ``sample`` replaces the
    verification result by the recorded (emitted tokens, accepted lengths).  All frames of a cohort are
    uploaded once, padded to the cohort's batch."""

    def __init__(self, trace: ReplayTrace, *, attention_dp: int, rank: int):
        if not trace.speculative:
            raise ValueError("a speculative replay needs a speculative trace")
        self.trace, self.attention_dp, self.rank = trace, attention_dp, rank
        self.cohorts, self.pending = {}, None

    def _prepare(self, cohort, repeat, batch, device):
        import torch

        ep = self.trace.episode(self.attention_dp, repeat, batch, self.rank)
        size, frames, width = ep["batch"], ep["frames"], ep["verify_width"]
        if not size or not frames:
            raise ReplayMismatch("an inactive replay rank has nothing to draft")

        def padded(name, cols, fill):
            rows = []
            for f in frames:
                vals = [list(v) + [fill] * (cols - len(v)) if cols else v for v in f[name]]
                rows.append(vals + ([[fill] * cols] if cols else [fill]) * (size - len(f["keys"])))
            return torch.tensor(rows, dtype=torch.int32, device=device)

        st = dict(episode=ep, index=0, draft_calls=0, sampler_calls=0, repeat=repeat, batch=batch,
                  tensors=dict(draft=padded("draft_tokens", width, 0), emitted=padded("emitted", width, -1),
                               lengths=padded("accept_lens", 0, 0)))
        self.cohorts[cohort] = st
        return st

    def draft(self, cohort, *, repeat: int, keys, seq_lens, steps: int, device="cpu", trace_sha256=None):
        """Scripted draft tokens int32 [len(keys), verify_width] of this step."""
        if trace_sha256 is not None and trace_sha256 != self.trace.sha256:
            raise ReplayMismatch("client and server replay traces differ")
        st = self.cohorts.get(cohort) or self._prepare(cohort, repeat, len(keys), device)
        if steps != st["episode"]["steps"]:
            raise ReplayMismatch("the engine's draft length differs from the recording")
        i = st["index"]
        if self.pending is not None or i >= len(st["episode"]["frames"]):
            raise ReplayMismatch("replay step overlaps or exceeds its recorded history")
        f = st["episode"]["frames"][i]
        if list(keys) != f["keys"] or list(seq_lens) != f["seq_lens"]:
            raise ReplayMismatch("replay request order or sequence positions differ from the recording")
        st["draft_calls"] += 1
        self.pending = (cohort, st, i, len(keys))
        return st["tensors"]["draft"][i, : len(keys)]

    def sample(self, natural_tokens, natural_lengths):
        """Replace the verification result: returns (emitted int32 [n, width] padded with -1, accepted int32 [n])."""
        if self.pending is None:
            return natural_tokens, natural_lengths
        cohort, st, i, n = self.pending
        forced = (st["tensors"]["emitted"][i, :n], st["tensors"]["lengths"][i, :n])
        if tuple(natural_tokens.shape) != tuple(forced[0].shape) or tuple(natural_lengths.shape) != tuple(forced[1].shape):
            raise ReplayMismatch("the engine's verification layout differs from the recording")
        st["sampler_calls"] += 1
        st["index"] += 1
        self.pending = None
        return forced

    def completed(self, cohort) -> bool:
        st = self.cohorts[cohort]
        return st["index"] == len(st["episode"]["frames"])

    def receipt(self, cohort) -> dict:
        st = self.cohorts[cohort]
        return dict(trace_sha256=self.trace.sha256, attention_dp=self.attention_dp, rank=self.rank, repeat=st["repeat"],
                    batch=st["batch"], frames=st["index"], expected_frames=len(st["episode"]["frames"]),
                    draft_calls=st["draft_calls"], sampler_calls=st["sampler_calls"], complete=self.completed(cohort),
                    forced_acceptance=True, natural_accuracy_claimed=False)


def force_logits(logits, replay_ids, positions):
    """Logits processor form of a replay: row i keeps only token ``replay_ids[i][positions[i]]`` (0.0, everything
    else -inf), so ANY sampler the engine runs afterwards selects the recorded token."""
    import torch

    if logits.ndim != 2 or len(replay_ids) != logits.shape[0] or len(positions) != logits.shape[0]:
        raise ReplayMismatch("forced-output batch differs from the logits")
    targets = []
    for ids, pos in zip(replay_ids, positions):
        if type(pos) is not int or not 0 <= pos < len(ids):
            raise ReplayMismatch("forced-output position exceeds the supplied history")
        tok = ids[pos]
        if type(tok) is not int or not 0 <= tok < logits.shape[1]:
            raise ReplayMismatch("forced-output token exceeds the vocabulary")
        targets.append(tok)
    logits.fill_(float("-inf"))
    logits.scatter_(1, torch.tensor(targets, device=logits.device, dtype=torch.long)[:, None], 0.0)
    return logits
