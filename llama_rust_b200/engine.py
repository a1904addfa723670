"""Continuous batching over one device-resident session: the batch formation of the reference's Engine
(langtax/src/engine.rs:487-494 `step`, :1132-1160 job collection, :1215-1274 one shared product for prompt chunks and
replayed tokens, :1307-1378 greedy sampling and the decode batch) with every forward pass, the paged KV pool and the
argmax on the device (llr_session_batch).

A step retires finished sequences, admits waiting ones into free slots, forwards one prompt chunk of every sequence that
is still reading its prompt together with the replay tokens of recomputed sequences as ONE ragged batch, then samples a
greedy token for every sequence whose logits are ready and forwards those tokens as a second batch.  A slot is a
sequence index of the session.  When the KV pool cannot take a batch, the most recently admitted other sequence loses its
blocks and is recomputed later from its prompt and the tokens it had generated (recompute preemption, engine.rs `on_cap`);
the tokens a sequence generates do not depend on that."""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from .executor import NativeCudaError, Session

ERR_OOM = 7


@dataclass
class EngineCfg:
    """EngineCfg (engine.rs:253-294), the knobs that concern batch formation."""
    max_seqs: int = 4
    prefill_chunk: int = 0      # prompt tokens per sequence per step; 0: the rest of the prompt
    eos: int | None = None
    decode_first: bool = False  # hold prompt chunks while any sequence decodes


@dataclass
class SeqOutput:
    prompt: list
    generated: list
    completion_tokens: int


@dataclass
class EngineStats:
    steps: int = 0
    gemm_tokens: int = 0    # tokens forwarded in a batch of two or more sequences
    gemm_peak: int = 0      # most tokens in one such batch
    serial_tokens: int = 0  # tokens forwarded one sequence at a time
    preempts: int = 0


@dataclass
class _Slot:
    id: int
    prompt: list
    n_predict: int
    generated: list = field(default_factory=list)
    completion_tokens: int = 0
    next_id: int | None = None  # greedy token of the logits of the last forwarded row, when they are current
    replay: int = 0             # generated tokens already back in the cache after a preemption
    done: bool = False
    order: int = 0


class Engine:
    def __init__(self, session: Session, cfg: EngineCfg | None = None):
        self.s, self.cfg = session, cfg or EngineCfg(max_seqs=session.n_seq)
        if self.cfg.max_seqs > session.n_seq:
            raise ValueError("the session has fewer sequences than max_seqs")
        self.slots: list[_Slot | None] = [None] * self.cfg.max_seqs
        self.wait: deque[_Slot] = deque()
        self.finished: dict[int, SeqOutput] = {}
        self.stats = EngineStats()
        self._next_id = 0
        self._admitted = 0

    # ---- public surface (engine.rs:457-560, :974) -----------------------------------------------------------
    def add(self, prompt, n_predict: int) -> int:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("empty prompt")
        sid = self._next_id
        self._next_id += 1
        self.wait.append(_Slot(sid, prompt, n_predict))
        return sid

    def step(self) -> int:
        n = self._retire() + self._admit()
        n += self._prefill_and_replay()
        n += self._decode_ready()
        self.stats.steps += 1
        return n

    def run(self) -> None:
        while not self.all_done():
            if self.step() == 0:
                raise RuntimeError("engine stall")
        self._retire()

    def all_done(self) -> bool:
        return not self.wait and all(s is None or s.done for s in self.slots)

    def active(self) -> int:
        return sum(s is not None for s in self.slots)

    def waiting(self) -> int:
        return len(self.wait)

    def take(self, sid: int) -> SeqOutput | None:
        return self.finished.pop(sid, None)

    def generated(self, sid: int):
        for s in list(self.slots) + list(self.wait):
            if s is not None and s.id == sid:
                return list(s.generated)
        return list(self.finished[sid].generated) if sid in self.finished else None

    # ---- one step ---------------------------------------------------------------------------------------------
    def _retire(self) -> int:
        n = 0
        for i, s in enumerate(self.slots):
            if s is not None and s.done:
                self.finished[s.id] = SeqOutput(s.prompt, s.generated, s.completion_tokens)
                self.s.seq_reset(i)
                self.slots[i] = None
                n += 1
        return n

    def _admit(self) -> int:
        n = 0
        while self.wait and None in self.slots:
            i = self.slots.index(None)
            s = self.wait.popleft()
            s.order = self._admitted
            self._admitted += 1
            self.slots[i] = s
            n += 1
        return n

    def _is_prefill(self, i: int) -> bool:
        s = self.slots[i]
        return s is not None and not s.done and self.s.seq_position(i) < len(s.prompt)

    def _is_decode(self, i: int) -> bool:
        s = self.slots[i]
        return (s is not None and not s.done and self.s.seq_position(i) >= len(s.prompt)
                and (s.next_id is not None or s.replay < len(s.generated)))

    def _forward(self, jobs) -> int:
        """jobs: [(slot, tokens, kind)]; one ragged batch.  kind: 'prompt', 'replay' or 'new'."""
        while jobs:
            try:
                nxt, _ = self.s.batch([(i, t) for i, t, _ in jobs])
                break
            except NativeCudaError as e:
                if e.code != ERR_OOM:
                    raise
                victim = self._preempt({i for i, _, _ in jobs})
                jobs = [j for j in jobs if j[0] != victim]
        else:
            return 1
        ntok = sum(len(t) for _, t, _ in jobs)
        if len(jobs) > 1:
            self.stats.gemm_tokens += ntok
            self.stats.gemm_peak = max(self.stats.gemm_peak, ntok)
        else:
            self.stats.serial_tokens += ntok
        for (i, t, kind), tok in zip(jobs, nxt):
            s = self.slots[i]
            if kind == "replay":
                s.replay += len(t)
            s.next_id = int(tok)
            # logits of a prompt prefix or of a prefix of the saved continuation are not the ones to sample from
            if self.s.seq_position(i) < len(s.prompt) or s.replay < len(s.generated):
                s.next_id = None
        return len(jobs)

    def _preempt(self, batch_slots) -> int:
        """Frees the cache of the most recently admitted live sequence (one outside the failing batch if there is any)."""
        live = [i for i, s in enumerate(self.slots) if s is not None and not s.done and self.s.seq_position(i) > 0]
        outside = [i for i in live if i not in batch_slots]
        pool = outside or [i for i in live if i in batch_slots]
        if not pool or (not outside and len(pool) == 1):
            raise NativeCudaError(ERR_OOM, "the KV pool cannot hold a single sequence of this batch")
        victim = max(pool, key=lambda i: self.slots[i].order)
        s = self.slots[victim]
        self.s.seq_reset(victim)
        s.replay, s.next_id = 0, None
        self.stats.preempts += 1
        return victim

    def _prefill_and_replay(self) -> int:
        hold = self.cfg.decode_first and any(self._is_decode(i) for i in range(len(self.slots)))
        jobs = []
        for i, s in enumerate(self.slots):
            if self._is_prefill(i):
                if not hold:
                    jobs.append((i, self.s.prompt_suffix(s.prompt, i, self.cfg.prefill_chunk), "prompt"))
            elif self._is_decode(i) and s.replay < len(s.generated):
                jobs.append((i, [s.generated[s.replay]], "replay"))
        return self._forward(jobs) if jobs else 0

    def _decode_ready(self) -> int:
        n, jobs = 0, []
        for i, s in enumerate(self.slots):
            if not self._is_decode(i) or s.replay < len(s.generated):
                continue
            if len(s.generated) >= s.n_predict:
                s.done = True
                n += 1
                continue
            tok = s.next_id
            s.completion_tokens += 1
            if self.cfg.eos is not None and tok == self.cfg.eos:
                s.done = True
                n += 1
                continue
            s.generated.append(tok)
            s.replay = len(s.generated)
            s.next_id = None
            if len(s.generated) >= s.n_predict:
                s.done = True
                n += 1
            else:
                jobs.append((i, [tok], "new"))
        return n + (self._forward(jobs) if jobs else 0)
