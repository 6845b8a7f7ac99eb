"""Integer sampler: drop-in for `bitexact.vllm_plugin.sampler` (src/bitexact/vllm_plugin/sampler.py): `integer_sample`
(:57-88), the `STASH` hand-over between `compute_logits` and the sampler (:41-54), `_strict` (:91-100) and the
logits processor `IntSampler` (:113-212) that forces vLLM's float sampler onto the integer-sampled token; and for
`bitexact.vllm_plugin.tri_logits.first_argmax` (vllm_plugin/tri_logits.py:97-100).

`IntSampler` needs vLLM only as a caller: it derives from vLLM's `LogitsProcessor` when that class can be imported
(the V2 model runner interface of the vLLM release the reference pins) and from `object` otherwise, and it reads the
request state and the step context through the same attributes (`max_num_reqs`, `prompt_len.np`, `idx_mapping_np`,
`seq_lens_upper_bound_np`, `expanded_idx_mapping`, `pos`). The host work is bookkeeping only; tokens come from the
sampler kernels (`bx_sample`)."""

import gc
import hashlib
import os
from fractions import Fraction

import numpy as np
import torch

from .. import _native as nv

try:                                                     # the base class only registers the hooks with vLLM
    from vllm.v1.worker.gpu.sample.logits_processor import LogitsProcessor as _Base
except Exception:                                        # vLLM absent or another release: same methods, no base
    _Base = object

FR = 24


def temp_ratio(t):
    """Float temperature -> (tn, td), T = tn / td with td <= 100; below 1e-5 (or None) is greedy = (0, 1)
    (src/bitexact/sampling.py:70-75)."""
    if t is None or t < 1e-5:
        return 0, 1
    f = Fraction(t).limit_denominator(100)
    return f.numerator, f.denominator


def sample_rows(li, rows, lnt, fr=FR):
    """li int64 [M, V] (unit column stride), rows int64 [M, 4] on the device = (seed, t, tn, td) per row
    (tn = 0: greedy) -> int64 [M] tokens. No host sync."""
    M, V = li.shape
    assert li.dtype == torch.int64 and li.stride(1) == 1
    tok = torch.empty(M, dtype=torch.long, device=li.device)
    if M:
        lib = nv.lib()
        scratch = torch.empty(max(1, lib.bx_sample_scratch_bytes(M, V)), dtype=torch.uint8, device=li.device)
        rc = lib.bx_sample(li.data_ptr(), li.stride(0), rows.data_ptr(), lnt.data_ptr(), scratch.data_ptr(),
                           tok.data_ptr(), M, V, fr, nv.stream())
        nv.check(rc, "bx_sample")
    return tok


def integer_sample(li, seeds, ts, temps, lnt, greedy=None, fr=FR):
    """li int64 [M, V]; per row seed, generated index t, (tn, td). Returns int64 [M] token ids."""
    rows = torch.tensor([[int(s), max(int(t), 0), int(tn), int(td)] for s, t, (tn, td) in zip(seeds, ts, temps)],
                        dtype=torch.long).reshape(-1, 4).to(li.device)
    return sample_rows(li, rows, lnt, fr)


def first_argmax(v):
    """Index of the first maximum of each row of int64 [M, V]."""
    rows = torch.zeros(v.shape[0], 4, dtype=torch.long, device=v.device)
    rows[:, 3] = 1
    return sample_rows(v, rows, rows, FR)


class _Stash:
    """What compute_logits leaves for the sampler of the same step (src/bitexact/vllm_plugin/sampler.py:41-54)."""
    logits = None            # int64 [rows, V] of the latest compute_logits (when no Head is kept)
    greedy = None            # int64 [rows]: first argmax of each logits row
    active = False           # set when the integer model is loaded in this process
    head = None              # tri_sample.Head of the latest compute_logits (the int64 logits are then not stored)
    strict = False           # this step: some request needs the real float logits
    gl = None                # (Head, one-hot logits, greedy) computed by a decode CUDA graph for this step
    gmode = (False, False)   # (strict, noisy) the replay hook chose for it
    sampler = None           # the IntSampler of the process
    fr = 16                  # fractional bits of the logits (int8 mode; 24 in exact mode)
    lnt = None               # the engine's ln table


STASH = _Stash()

_FLOAT_LOGIT_FIELDS = ("presence_penalty", "frequency_penalty", "logit_bias", "allowed_token_ids", "bad_words",
                       "bad_words_token_ids", "min_tokens", "logits_processors", "extra_args")


def _strict(sp):
    """Does the request read or edit vLLM's float logits before the draw (log-probs, penalties, bias, allowed / bad
    words, min_tokens, structured output, extra processors)? Only then are real float logits produced
    (src/bitexact/vllm_plugin/sampler.py:91-100)."""
    if sp.logprobs is not None or getattr(sp, "prompt_logprobs", None) is not None:
        return True
    if getattr(sp, "repetition_penalty", 1.0) != 1.0 or getattr(sp, "structured_outputs", None) is not None:
        return True
    return any(bool(getattr(sp, f, None)) for f in _FLOAT_LOGIT_FIELDS)


def _request_state(view):
    """The model runner's request table behind the processor's view (they share `total_len`), or False: vLLM gives
    a logits processor no callback when a request finishes (src/bitexact/vllm_plugin/sampler.py:103-110)."""
    for o in gc.get_referrers(view.total_len):
        if getattr(o, "total_len", None) is view.total_len and hasattr(o, "req_id_to_index"):
            return o
    return False


class IntSampler(_Base):
    """Per request slot: seed, temperature ratio and whether the request is strict; per step: integer tokens for all
    logits rows, written into vLLM's float logits as 0 at the token and -inf elsewhere, so that temperature, top-k /
    top-p and vLLM's own random draw can only return that token. No host-device synchronisation in plain decoding:
    rows map to slots through vLLM's host copies, t = sequence length - prompt length."""

    def __init__(self, vllm_config, req_states):
        self.rs = req_states
        n = req_states.max_num_reqs
        self.seed = np.zeros(n, dtype=np.int64)
        self.tn = np.zeros(n, dtype=np.int64)            # T = tn / td, tn = 0: greedy
        self.td = np.ones(n, dtype=np.int64)
        self.strict = np.zeros(n, dtype=bool)
        self.log = os.environ.get("BITEXACT_HASH_LOG")
        self.table = None                                # request table of the runner: None = not looked up yet
        self.lp = None                                   # RL runs: list collecting (seeds, ts, log p) per step
        STASH.sampler = self

    def add_request(self, req_idx, sampling_params):
        if not STASH.active:
            return False
        self.seed[req_idx] = int(sampling_params.seed or 0)
        self.tn[req_idx], self.td[req_idx] = temp_ratio(sampling_params.temperature)
        self.strict[req_idx] = bool(_strict(sampling_params) or self.log)
        return bool(self.strict[req_idx] or self.tn[req_idx] != 0)

    def _running(self):
        if self.table is None:
            self.table = _request_state(self.rs)
        if self.table is False:
            return None                                  # unknown: every slot counts (slower, never wrong)
        d = self.table.req_id_to_index
        return np.fromiter(d.values(), dtype=np.intp, count=len(d))

    def any_noisy(self):
        """Does a running request sample with a temperature?"""
        run = self._running()
        return True if run is None else bool(self.tn[run].any())

    def any_strict(self):
        """Does a running request need real float logits? vLLM's warm-up requests leave flags in free slots, so only
        running slots count when the runner's table is known."""
        run = self._running()
        return bool(self.strict.any()) if run is None else bool(self.strict[run].any())

    def apply(self, logits, ctx):
        if not STASH.active:
            return logits
        from . import tri_sample
        head = STASH.head
        li = None if head is not None else STASH.logits
        assert head is not None or li is not None, "compute_logits left no integer logits"
        n = head.R if head is not None else li.shape[0]
        assert n == logits.shape[0], "integer logits rows != vLLM rows"
        slots = ctx.idx_mapping_np
        plen = self.rs.prompt_len.np
        if len(slots) == n:                              # one logits row per request
            rows = np.asarray(slots, dtype=np.intp)
            ts = ctx.seq_lens_upper_bound_np[:n].astype(np.int64) - plen[rows].astype(np.int64)
        else:
            # Speculative decoding: 1 + k rows per request; how many drafts were accepted is only known on the device,
            # so the generated index of a row comes from its position (the row at position p samples token p + 1).
            rows = ctx.expanded_idx_mapping.cpu().numpy().astype(np.intp)
            ts = ctx.pos.cpu().numpy().astype(np.int64) + 1 - plen[rows].astype(np.int64)
        st = np.stack([self.seed[rows], np.maximum(ts, 0), self.tn[rows], self.td[rows]], 1)
        if head is not None:                             # one pass over the head's output, writes vLLM's rows too
            assert logits.is_contiguous()
            y = tri_sample.noisy(head, st, STASH.lnt, out=logits)
        else:
            y = sample_rows(li, torch.from_numpy(st).to(li.device, non_blocking=True), STASH.lnt, STASH.fr)
            logits.fill_(float("-inf"))
            logits.scatter_(1, y[:, None], 0.0)
        if self.lp is not None or self.log:
            full = head.logits() if li is None else li
            if self.lp is not None:
                from .rl import int_logp
                self.lp.append((self.seed[rows].copy(), ts, int_logp(full, y, STASH.lnt, STASH.fr)))
            if self.log:
                self._log(full, self.seed[rows].tolist(), ts.tolist(), y)
        return logits

    def _log(self, li, seeds, ts, y):
        """One line "seed t sha16 token" per sampled row (rows of unfinished prompt chunks, t < 0, are left out)."""
        rows, ys = li.cpu().numpy(), y.tolist()
        with open(self.log, "a") as f:
            for r, (seed, t) in enumerate(zip(seeds, ts)):
                if t >= 0:
                    f.write("%d %d %s %d\n" % (seed, t, hashlib.sha256(rows[r].tobytes()).hexdigest()[:16], ys[r]))
