"""Host side of the vLLM sampler hook (IntSampler): temperature ratios, the strict-request rule and the per-slot
bookkeeping, against fakes of vLLM's request state (no vLLM, no GPU). Follows the behaviour documented in the
reference's src/bitexact/vllm_plugin/sampler.py:1-26, 91-151."""

from types import SimpleNamespace

import numpy as np

from bitexact_llm_b200.vllm_plugin import sampler as S


def _sp(**kw):
    base = dict(seed=None, temperature=0.0, logprobs=None, prompt_logprobs=None, presence_penalty=0.0,
                frequency_penalty=0.0, repetition_penalty=1.0, logit_bias=None, allowed_token_ids=None, bad_words=None,
                min_tokens=0, structured_outputs=None, logits_processors=None, extra_args=None)
    base.update(kw)
    return SimpleNamespace(**base)


class _Table:
    """Stands for the model runner's request table: shares `total_len` with the processor's view."""

    def __init__(self, total_len):
        self.total_len = total_len
        self.req_id_to_index = {}


def _states(n=8):
    total = np.zeros(n, dtype=np.int64)
    view = SimpleNamespace(max_num_reqs=n, total_len=total, prompt_len=SimpleNamespace(np=np.zeros(n, dtype=np.int32)))
    return view, _Table(total)


def test_temp_ratio():
    assert S.temp_ratio(None) == (0, 1) and S.temp_ratio(0.0) == (0, 1) and S.temp_ratio(9e-6) == (0, 1)
    assert S.temp_ratio(0.7) == (7, 10) and S.temp_ratio(1.0) == (1, 1) and S.temp_ratio(1.3) == (13, 10)
    assert S.temp_ratio(0.333) == (1, 3) and S.temp_ratio(2.5) == (5, 2)
    tn, td = S.temp_ratio(0.123456)
    assert td <= 100 and abs(tn / td - 0.123456) < 1e-3


def test_strict_rule():
    assert not S._strict(_sp())
    assert not S._strict(_sp(temperature=0.7, seed=5))
    for kw in (dict(logprobs=0), dict(prompt_logprobs=1), dict(presence_penalty=0.1), dict(frequency_penalty=-0.2),
               dict(repetition_penalty=1.1), dict(logit_bias={3: 1.0}), dict(allowed_token_ids=[1, 2]),
               dict(bad_words=["x"]), dict(min_tokens=2), dict(structured_outputs=object()),
               dict(logits_processors=[object()]), dict(extra_args={"bitexact_score_from": 4})):
        assert S._strict(_sp(**kw)), kw


def test_slots_and_running_requests():
    view, table = _states()
    old = S.STASH.active
    try:
        S.STASH.active = False
        smp = S.IntSampler(None, view)
        assert S.STASH.sampler is smp
        assert smp.add_request(0, _sp(temperature=0.7)) is False         # integer model not loaded: hook stays off
        S.STASH.active = True
        assert smp.add_request(1, _sp()) is False                         # greedy, not strict: nothing to do per step
        assert smp.add_request(2, _sp(temperature=0.7, seed=11)) is True
        assert smp.add_request(3, _sp(logprobs=5)) is True
        assert (smp.seed[2], smp.tn[2], smp.td[2]) == (11, 7, 10) and smp.tn[1] == 0 and smp.strict[3]
        # free slots keep the flags of finished (or warm-up) requests: only running slots count
        table.req_id_to_index = {"a": 1}
        assert not smp.any_noisy() and not smp.any_strict()
        table.req_id_to_index = {"a": 1, "b": 2}
        assert smp.any_noisy() and not smp.any_strict()
        table.req_id_to_index = {"c": 3}
        assert not smp.any_noisy() and smp.any_strict()
        # a runner whose table cannot be found: every flag counts
        lost = S.IntSampler(None, SimpleNamespace(max_num_reqs=4, total_len=np.zeros(4, dtype=np.int64),
                                                  prompt_len=SimpleNamespace(np=np.zeros(4, dtype=np.int32))))
        assert lost.any_noisy() and not lost.any_strict()
        lost.add_request(0, _sp(min_tokens=3))
        assert lost.any_strict()
        del table
    finally:
        S.STASH.active = old
        S.STASH.sampler = None
