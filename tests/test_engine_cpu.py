"""The batch scheduler (llama_rust_b200/engine.py, the reference's Engine::step: langtax/src/engine.rs:487-494) on CPU,
against a stand-in for the device session: a toy model whose next token is a fixed function of the whole sequence so
far, over a block pool of limited size that refuses a batch with the library's out-of-blocks status.  What is checked is
host logic only: admission, prompt chunks, mixed prompt and decode batches, replay after a preemption, eos, decode_first."""
import pytest

from llama_rust_b200.engine import ERR_OOM, Engine, EngineCfg
from llama_rust_b200.executor import NativeCudaError


def _next(tokens):
    h = 17
    for t in tokens:
        h = (h * 31 + t + 7) % 1009
    return h % 50


class FakeSession:
    """The part of Session the Engine uses: batch, seq_position, seq_reset, prompt_suffix; blocks of `block` positions."""

    def __init__(self, n_seq, kv_blocks, block=2):
        self.n_seq, self.free, self.block = n_seq, kv_blocks, block
        self.ids = [[] for _ in range(n_seq)]
        self.held = [0] * n_seq
        self.batches = []

    def seq_position(self, q):
        return len(self.ids[q])

    def seq_reset(self, q):
        self.free += self.held[q]
        self.held[q], self.ids[q] = 0, []

    def prompt_suffix(self, tokens, seq=0, max_suffix=0):
        have = self.ids[seq]
        lcp = 0
        while lcp < len(have) and lcp < len(tokens) and have[lcp] == tokens[lcp]:
            lcp += 1
        keep = len(tokens) - 1 if lcp == len(tokens) else lcp
        del self.ids[seq][keep:]
        rest = list(tokens[keep:])
        return rest[:max_suffix] if max_suffix else rest

    def batch(self, groups, want_logits=False):
        assert len({q for q, _ in groups}) == len(groups) and all(len(t) > 0 for _, t in groups)
        need = []
        for q, t in groups:
            blocks = -(-(len(self.ids[q]) + len(t)) // self.block)
            need.append(max(0, blocks - self.held[q]))
        if sum(need) > self.free:
            raise NativeCudaError(ERR_OOM, "no free block")
        out = []
        for (q, t), n in zip(groups, need):
            self.held[q] += n
            self.free -= n
            self.ids[q].extend(t)
            out.append(_next(self.ids[q]))
        self.batches.append([(q, len(t)) for q, t in groups])
        return out, None


def _alone(prompt, n):
    seq, out = list(prompt), []
    for _ in range(n):
        out.append(_next(seq))
        seq.append(out[-1])
    return out


def test_mixed_batches_generate_the_sequential_continuations():  # native_cuda_parity.rs:258-289
    prompts = [[1, 2, 3], [1, 2, 4, 5], [1, 2]]
    s = FakeSession(2, 64)
    e = Engine(s, EngineCfg(max_seqs=2, prefill_chunk=2))
    a, b = e.add(prompts[0], 4), e.add(prompts[1], 4)
    assert e.step() > 0
    c = e.add(prompts[2], 4)
    assert e.waiting() == 1 and e.active() == 2
    e.run()
    assert e.stats.gemm_peak > 1 and e.all_done()
    for sid, p in zip((a, b, c), prompts):
        out = e.take(sid)
        assert out.prompt == p and out.generated == _alone(p, 4) and out.completion_tokens == 4
    assert e.take(a) is None
    # chunks of at most two prompt tokens per sequence, and a batch that mixes a prompt chunk with a decode token
    assert all(n <= 2 for batch in s.batches for _, n in batch)
    assert any(len(batch) == 2 and {n for _, n in batch} == {1, 2} for batch in s.batches)
    assert s.free == 64  # every block went back


def test_preemption_recomputes_and_outputs_do_not_change():
    prompts = [[1, 2, 3, 4, 5, 6], [7, 8, 9], [3, 1, 4, 1, 5, 9, 2, 6]]
    s = FakeSession(3, 14)  # three sequences need up to 9 blocks each
    e = Engine(s, EngineCfg(max_seqs=3, prefill_chunk=4))
    ids = [e.add(p, 10) for p in prompts]
    e.run()
    assert e.stats.preempts > 0
    for sid, p in zip(ids, prompts):
        assert e.take(sid).generated == _alone(p, 10)


def test_a_pool_too_small_for_one_sequence_is_an_error_not_a_loop():
    s = FakeSession(2, 2)
    e = Engine(s, EngineCfg(max_seqs=2))
    e.add([1, 2, 3, 4, 5, 6], 4)
    with pytest.raises(NativeCudaError) as err:
        e.run()
    assert err.value.code == ERR_OOM


def test_eos_and_decode_first():
    p0, p1 = [5, 6, 7, 8, 9], [2, 3]
    want0 = _alone(p0, 12)
    eos = want0[4]
    cut = want0.index(eos)
    s = FakeSession(2, 64)
    e = Engine(s, EngineCfg(max_seqs=2, prefill_chunk=2, eos=eos, decode_first=True))
    b = e.add(p1, 12)
    e.step()
    e.step()                      # sequence b is decoding by now
    a = e.add(p0, 12)
    before = len(s.batches)
    while e.generated(b) is not None and len(e.generated(b)) < 11 and not e.all_done():
        e.step()
    held = s.batches[before:len(s.batches) - 1]
    # decode_first: while b decodes, a's prompt chunks are held back: only single decode tokens were forwarded
    assert held and all(n == 1 for batch in held for _, n in batch)
    e.run()
    out = e.take(a)
    assert out.generated == want0[:cut] and out.completion_tokens == cut + 1
    wb = _alone(p1, 12)
    assert e.take(b).generated == (wb[:wb.index(eos)] if eos in wb else wb)


def test_validation():
    s = FakeSession(2, 8)
    with pytest.raises(ValueError):
        Engine(s, EngineCfg(max_seqs=3))
    e = Engine(s)
    with pytest.raises(ValueError):
        e.add([], 4)
