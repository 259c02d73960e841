"""Continuous batching above the step function.

The scheduler admits requests, cuts prompts into portions under a per-step token budget,
decodes, finishes and frees.  Names follow the reference (``ContinuousScheduler``,
``Request``, ``GenerationResult``, ``max_concurrent``, ``decode_headroom_blocks``,
``chunk_size``, ``trace_out``: ``scheduler/continuous_scheduler.py:168-177``,
``scheduler/request_state.py:30-70``); the policy differs where the reference leaves room:

* **Admission** is first come, first served, while fewer than ``max_concurrent`` requests
  are live and the free pages cover the whole prompt plus ``decode_headroom_blocks``
  (the reference's rule, ``:711-760``).  A prompt that could never fit the pool is
  finished as ``"cancelled"``.
* **Token budget.**  A step holds at most ``max_tokens_per_step`` tokens: every decoding
  request brings one, the rest of the budget goes to prefilling requests in admission
  order, each at most ``chunk_size`` tokens, the last one cut to fit (the reference has a
  per-request chunk only, ``:1009-1010``).
* **When pages run out.**  The step is planned before anything is launched.  If the pages
  for it are not there, prompt portions are shrunk first, from the youngest; if the
  decoding tokens alone do not fit, the youngest live request is preempted *by recompute*:
  its pages are freed and it goes back to the head of the queue with its prompt plus what
  it has generated, keeping its sampling seed and token count, so it continues the same
  sequence later.  (The reference cancels the youngest request instead, ``:373-445``.)  A
  request that cannot fit even alone is finished as ``"cancelled"``.
* **Faults.**  With every step's tokens the scheduler reads the runner's health word (set by
  a kernel that gave up a bounded wait).  If it is set, the step's requests are finished as
  ``"cancelled"`` with their pages given back, the runner is reset, and ``EngineFaultError``
  is raised; nothing sampled from that step is handed out.
* **Finishing.**  ``"stop"`` when the sampled id is an end-of-sequence id (it is not
  emitted), ``"length"`` after ``max_tokens`` tokens or at the model's last position.
  A finished request's pages go back before the next step is planned.
"""

from __future__ import annotations

import collections
import dataclasses
import enum
import json
import threading
import time
from typing import Callable, Hashable, Sequence

from ..cache.manager import CacheManager, OutOfPages
from ..sampling.params import SamplingParams
from ..sampling.sampler import default_seed
from .step import StepEntry


class EngineNotRunningError(RuntimeError):
    pass


class EngineFaultError(RuntimeError):
    """A step's kernels reported that they gave up waiting for their copies: the tokens of that
    step are worthless.  The step's requests are finished as ``"cancelled"``, the runner's
    health is reset, and the error is raised to whoever drives the engine."""


@dataclasses.dataclass
class Request:
    """A generation request: ``prompt`` is a list of token ids (or text, when the scheduler
    has a tokenizer)."""

    prompt: Sequence[int] | str
    sampling_params: SamplingParams = dataclasses.field(default_factory=SamplingParams)
    max_tokens: int = 16


@dataclasses.dataclass
class GenerationResult:
    text: str
    tokens: list[int]
    finish_reason: str
    prompt_tokens: int


class RequestState(enum.Enum):
    WAITING = "waiting"
    PREFILLING = "prefilling"
    DECODING = "decoding"
    DONE = "done"


@dataclasses.dataclass(frozen=True)
class SchedulerLoad:
    """The five numbers of the reference's ``load_stats`` (``scheduler/load.py``)."""

    num_waiting: int
    num_running: int
    kv_cache_usage: float
    block_size: int
    num_blocks: int


class RunningRequest:
    """Scheduler-side record of one request."""

    def __init__(self, rid: int, request: Request, prompt_ids: list[int], seed: int) -> None:
        self.rid = rid
        self.request = request
        self.prompt_ids = prompt_ids            # the caller's prompt
        self.feed = list(prompt_ids)            # tokens to prefill (prompt, plus generated after a preemption)
        self.fed = 0                            # tokens of ``feed`` already in the cache
        self.generated: list[int] = []
        self.next_token: int | None = None      # sampled, not yet fed
        self.state = RequestState.WAITING
        self.finish_reason: str | None = None
        self.seed = seed
        self.admitted_at = -1                   # admission order (for "youngest")
        self.preemptions = 0
        self.done = threading.Event()
        self.on_token: Callable[[int], None] | None = None
        self.cancel_requested = False
        self.in_flight_after_done = False       # finished while a step launched ahead still writes its pages

    def result(self, detokenize=None) -> GenerationResult:
        text = detokenize(self.generated) if detokenize else ""
        return GenerationResult(text=text, tokens=list(self.generated),
                                finish_reason=self.finish_reason or "", prompt_tokens=len(self.prompt_ids))


class RequestHandle:
    def __init__(self, scheduler: "ContinuousScheduler", rr: RunningRequest) -> None:
        self._scheduler = scheduler
        self._rr = rr

    def wait(self, timeout: float | None = None) -> GenerationResult:
        deadline = None if timeout is None else time.time() + timeout
        while not self._rr.done.wait(0.05):
            if self._scheduler._crashed is not None:
                raise EngineNotRunningError(f"the engine stopped: {self._scheduler._crashed!r}")
            if deadline is not None and time.time() > deadline:
                raise TimeoutError("request did not finish in time")
        return self._rr.result(self._scheduler._detokenize)

    def cancel(self) -> None:
        self._scheduler._cancel(self._rr)

    @property
    def finished(self) -> bool:
        return self._rr.done.is_set()


@dataclasses.dataclass
class _InFlightStep:
    """A decode step that has been launched and not yet read back."""

    entries: list
    owners: list                      # RunningRequest of each entry
    sampled: object                   # the sampler's output on the device, one id per entry
    host: object                      # the same ids on their way to (pinned) host memory
    ready: object                     # event recorded after that copy (None: the copy was synchronous)
    t0: float
    health: object = None             # the runner's health word on its way to the host (None: the runner has none)


class ContinuousScheduler:
    def __init__(
        self,
        runner,
        *,
        max_concurrent: int = 16,
        decode_headroom_blocks: int = 8,
        chunk_size: int | None = None,
        max_tokens_per_step: int = 2048,
        eos_token_ids: Sequence[int] = (),
        sampler=None,
        tokenizer=None,
        trace_out: str | None = None,
        lookahead: bool | None = None,
    ) -> None:
        # chunk_size: the most prompt tokens one request feeds in a step (the reference's option,
        # whose default there is 256).  None: whatever the step's token budget leaves, so prompts
        # are fed oldest first and whole where they fit.  The budget, not the chunk, bounds how
        # long a step keeps the decoding requests waiting; a smaller chunk only shortens steps
        # that few prompts share, at the price of later first tokens (1,024-token prompts, 16
        # together: median first token after 117 ms of steps instead of 158).
        if chunk_size is None:
            chunk_size = max_tokens_per_step
        if max_concurrent <= 0 or chunk_size <= 0 or max_tokens_per_step <= 0:
            raise ValueError("max_concurrent, chunk_size and max_tokens_per_step must be positive")
        self.runner = runner
        self.cache: CacheManager = runner.cache
        self.max_concurrent = min(max_concurrent, self.cache.max_requests)
        self.decode_headroom_blocks = decode_headroom_blocks
        self.chunk_size = chunk_size
        self.max_tokens_per_step = max_tokens_per_step
        self.eos_token_ids = frozenset(int(t) for t in eos_token_ids)
        self.max_positions = getattr(runner, "max_positions", None)
        if sampler is None:
            from ..sampling.sampler import DeviceSampler

            sampler = DeviceSampler(runner.device)
        self.sampler = sampler
        self.tokenizer = tokenizer
        self._detokenize = tokenizer.decode if tokenizer is not None else None
        self.trace_out = trace_out
        self._trace: list[dict] = []
        self._waiting: collections.deque[RunningRequest] = collections.deque()
        self._live: list[RunningRequest] = []
        self._lock = threading.Lock()
        self._next_rid = 0
        self._admissions = 0
        self._thread: threading.Thread | None = None
        self._stop = threading.Event()
        self._wake = threading.Event()      # set by submit: an idle engine thread starts at once
        self._crashed: BaseException | None = None
        self.steps = 0
        self.tokens_generated = 0
        self.preemptions = 0
        self.last_step_entries: list[StepEntry] = []
        # Decode look-ahead: while every live request is decoding and nobody waits, the next
        # step is launched from the sampler's device output before the host reads it, so the
        # GPU never idles behind the host's bookkeeping.  A request that turns out to have
        # finished (a stop token) has then one token computed in vain; its pages are given
        # back when that step has been read.  Needs a runner that takes device tokens.
        if lookahead is None:
            lookahead = bool(getattr(runner, "device_token_feedback", False))
        self.lookahead = lookahead
        self._inflight: _InFlightStep | None = None
        self.wasted_tokens = 0

    # ------------------------------------------------------------------ public

    def submit(self, request: Request, on_token: Callable[[int], None] | None = None) -> RequestHandle:
        prompt = request.prompt
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer; pass token ids instead")
            prompt_ids = list(self.tokenizer.encode(prompt))
        else:
            prompt_ids = [int(t) for t in prompt]
        if request.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        with self._lock:
            rid = self._next_rid
            self._next_rid += 1
            seed = request.sampling_params.seed
            rr = RunningRequest(rid, request, prompt_ids, default_seed(rid) if seed is None else seed)
            rr.on_token = on_token
            if not prompt_ids:
                self._finish(rr, "stop")        # nothing to condition on (reference :703-707)
            elif self.max_positions is not None and len(prompt_ids) >= self.max_positions:
                self._finish(rr, "cancelled")   # no position left to generate at
            else:
                self._waiting.append(rr)
        self._wake.set()
        return RequestHandle(self, rr)

    def run(self, request: Request) -> GenerationResult:
        """Submit and wait (drives the engine itself when no engine thread runs)."""
        handle = self.submit(request)
        if self._thread is None:
            self.run_until_done()
        return handle.wait()

    def generate(self, requests: Sequence[Request]) -> list[GenerationResult]:
        handles = [self.submit(r) for r in requests]
        if self._thread is None:
            self.run_until_done()
        return [h.wait() for h in handles]

    def run_until_done(self) -> None:
        while self.step():
            pass

    def start(self, capture_decode_steps: bool = True) -> None:
        """Run the engine loop on a thread of its own until ``stop``.  A runner that replays
        captured decode steps captures those of every batch size up to ``max_concurrent`` first
        (under a second in all), so that no request meets a capture in the middle of serving."""
        if self._thread is not None:
            return
        self._stop.clear()
        if capture_decode_steps and hasattr(self.runner, "capture_decode_steps") and not self._live:
            self.runner.capture_decode_steps(self.max_concurrent)

        def loop() -> None:
            try:
                while not self._stop.is_set():
                    if not self.step():
                        self._wake.wait(0.005)
                        self._wake.clear()
            except BaseException as e:  # noqa: BLE001
                self._crashed = e
                raise

        self._thread = threading.Thread(target=loop, name="mini-infer-engine", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        self._drain()
        with self._lock:
            for rr in list(self._live):
                self._release(rr)
                self._finish(rr, "cancelled")
            self._live.clear()
            while self._waiting:
                self._finish(self._waiting.popleft(), "cancelled")
        if self.trace_out:
            with open(self.trace_out, "w", encoding="utf-8") as f:
                json.dump({"traceEvents": self._trace}, f)

    def has_prefill_work(self) -> bool:
        """True while a request waits for admission or still has prompt tokens to feed."""
        with self._lock:
            return bool(self._waiting) or any(r.state is RequestState.PREFILLING for r in self._live)

    def load_stats(self) -> SchedulerLoad:
        with self._lock:
            return SchedulerLoad(
                num_waiting=len(self._waiting), num_running=len(self._live),
                kv_cache_usage=self.cache.usage(), block_size=self.cache.page_size,
                num_blocks=sum(p.num_pages for p in self.cache.pools),
            )

    # ------------------------------------------------------------------ one engine step

    def step(self) -> bool:
        """Admit, plan, run one batch, sample, finish.  False when there is nothing to do.
        One call hands out one batch's tokens, whether or not a step was launched ahead."""
        if self._inflight is not None:
            cur, self._inflight = self._inflight, None
            self._inflight = self._launch_ahead(cur)
            self._collect(cur)
            return True
        with self._lock:
            for rr in [r for r in self._live if r.cancel_requested]:
                self._retire(rr, "cancelled")
            for rr in [r for r in self._waiting if r.cancel_requested]:
                self._waiting.remove(rr)
                self._finish(rr, "cancelled")
            self._admit()
            entries, owners = self._plan()
        if not entries:
            return False
        if self.lookahead and self._pure_decode(entries, owners):
            cur = self._launch(entries, owners, None)
            self._inflight = self._launch_ahead(cur)
            self._collect(cur)
            return True
        t0 = time.time()
        result = self.runner.step(entries)
        self.last_step_entries = entries
        self.steps += 1
        wanting = [rr for rr, e in zip(owners, entries) if e.want]
        if wanting:
            ids = self.sampler.sample(
                result.logits,
                [rr.request.sampling_params for rr in wanting],
                [rr.seed for rr in wanting],
                [len(rr.generated) for rr in wanting],
            )
            health = self._queue_health_read()
            ids = [int(t) for t in (ids.tolist() if hasattr(ids, "tolist") else ids)]
        else:
            # nothing is read back from this step, so nothing waits for it here; the health
            # word stays set once it is, and the next step that hands out tokens reads it
            health, ids = None, []
        self._check_health(health, owners)
        emitted: list = []
        with self._lock:
            for rr, e in zip(owners, entries):
                if rr.state is RequestState.PREFILLING:
                    rr.fed += len(e.tokens)
                    if rr.fed == len(rr.feed):
                        rr.state = RequestState.DECODING
                else:
                    rr.next_token = None
            for rr, tok in zip(wanting, ids):
                self._consume(rr, tok, emitted=emitted)
            if self.trace_out is not None:
                n_pre = sum(1 for e in entries if len(e.tokens) > 1)
                phase = "decode" if n_pre == 0 else ("prefill" if n_pre == len(entries) else "mixed")
                self._trace.append({
                    "name": "step", "ph": "X", "pid": 0, "tid": 0, "ts": t0 * 1e6,
                    "dur": (time.time() - t0) * 1e6,
                    "args": {"B": len(entries), "phase": phase,
                             "total_q": sum(len(e.tokens) for e in entries)},
                })
        self._emit(emitted)
        return True

    # ------------------------------------------------------------------ health

    def _queue_health_read(self):
        """Start a copy of the runner's health word to the host, behind the step just launched
        (None when the runner has no such word)."""
        word_of = getattr(self.runner, "health_word", None)
        word = word_of() if word_of is not None else None
        if word is None:
            return None
        if getattr(word, "is_cuda", False):
            import torch

            host = torch.empty(word.shape, dtype=word.dtype, pin_memory=True)
            host.copy_(word, non_blocking=True)
            return host
        return word

    def _check_health(self, health, owners) -> None:
        """Called once the step's results are on the host.  A set word means that the step's
        tokens are worthless: its requests end as ``"cancelled"`` and the error goes up."""
        if health is None or not int(health[0]):
            return
        self._drain(check=False)
        with self._lock:
            for rr in owners:
                rr.in_flight_after_done = False
                if rr.state is not RequestState.DONE:
                    self._retire(rr, "cancelled")
                else:
                    self._release(rr)
        reset = getattr(self.runner, "reset_health", None)
        if reset is not None:
            reset()
        raise EngineFaultError("a kernel gave up waiting for its copies; the step's tokens were discarded, "
                               f"{len(owners)} requests were cancelled and the runner was reset")

    def _emit(self, emitted) -> None:
        """Streaming callbacks run outside the scheduler's lock: a callback may cancel its own
        request, submit another one or ask for the load without deadlocking the engine."""
        for callback, token in emitted:
            callback(token)

    # ------------------------------------------------------------------ decode look-ahead

    def _pure_decode(self, entries, owners) -> bool:
        with self._lock:
            return (not self._waiting and len(owners) == len(self._live)
                    and all(rr.state is RequestState.DECODING and len(e.tokens) == 1
                            for rr, e in zip(owners, entries)))

    def _launch(self, entries, owners, device_tokens) -> _InFlightStep:
        """Put a decode step and its sampling on the stream; start the copy of the sampled ids
        to the host; do not wait for any of it."""
        import torch

        t0 = time.time()
        if device_tokens is None:
            result = self.runner.step(entries)
        else:
            result = self.runner.step(entries, device_tokens=device_tokens)
        self.last_step_entries = entries
        self.steps += 1
        # the draw index counts the tokens a request has been given, the one in flight included
        ahead = 0 if device_tokens is None else 1
        sampled = self.sampler.sample(
            result.logits,
            [rr.request.sampling_params for rr in owners],
            [rr.seed for rr in owners],
            [len(rr.generated) + ahead for rr in owners],
        )
        ready = None
        if isinstance(sampled, torch.Tensor) and sampled.is_cuda:
            host = torch.empty(sampled.shape, dtype=sampled.dtype, pin_memory=True)
            host.copy_(sampled, non_blocking=True)
            health = self._queue_health_read()
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(sampled.device))
        else:
            host = sampled
            health = self._queue_health_read()
        with self._lock:
            for rr in owners:
                rr.next_token = None
        return _InFlightStep(entries=entries, owners=owners, sampled=sampled, host=host, ready=ready, t0=t0,
                             health=health)

    def _launch_ahead(self, cur: _InFlightStep) -> _InFlightStep | None:
        """The step after ``cur`` for the requests that are known to go on (none has reached
        its length), fed from ``cur``'s sampled ids on the device; None when the batch is
        about to change (someone waits, prefills or wants out) or pages are short: the
        ordinary path then decides with everything read back."""
        import torch

        if not self.lookahead or not isinstance(cur.sampled, torch.Tensor):
            return None
        with self._lock:
            if self._waiting or any(rr.cancel_requested or rr.state is not RequestState.DECODING
                                    for rr in self._live):
                return None
            keep: list[int] = []
            for i, rr in enumerate(cur.owners):
                if rr.in_flight_after_done or rr.state is not RequestState.DECODING:
                    continue
                if len(rr.generated) + 1 >= rr.request.max_tokens:
                    continue                     # cur's token is its last
                if self.max_positions is not None and self.cache.length(rr.rid) + 1 > self.max_positions:
                    continue
                keep.append(i)
            if not keep or not self.cache.can_append([(cur.owners[i].rid, 1) for i in keep]):
                return None
            owners = [cur.owners[i] for i in keep]
        if len(keep) == len(cur.owners):
            tokens = cur.sampled
        else:
            index = torch.tensor(keep, dtype=torch.int64)
            if cur.sampled.is_cuda:
                index = index.pin_memory().to(cur.sampled.device, non_blocking=True)
            tokens = cur.sampled.index_select(0, index)
        entries = [StepEntry(rr.rid, [0], [0]) for rr in owners]
        return self._launch(entries, owners, tokens.to(torch.int32))

    def _collect(self, cur: _InFlightStep, check: bool = True) -> None:
        """Read a launched step's tokens and hand them to their requests."""
        if cur.ready is not None:
            cur.ready.synchronize()
        if check:
            self._check_health(cur.health, cur.owners)
        ids = [int(t) for t in (cur.host.tolist() if hasattr(cur.host, "tolist") else cur.host)]
        nxt = self._inflight
        ahead = set(id(rr) for rr in nxt.owners) if nxt is not None else set()
        emitted: list = []
        with self._lock:
            for rr, tok in zip(cur.owners, ids):
                if rr.in_flight_after_done:
                    # the step that was launched before its end was known: nothing to keep,
                    # and nothing writes its pages any more
                    rr.in_flight_after_done = False
                    self.wasted_tokens += 1
                    self._release(rr)
                    continue
                self._consume(rr, tok, still_in_flight=id(rr) in ahead, emitted=emitted)
            if self.trace_out is not None:
                self._trace.append({
                    "name": "step", "ph": "X", "pid": 0, "tid": 0, "ts": cur.t0 * 1e6,
                    "dur": (time.time() - cur.t0) * 1e6,
                    "args": {"B": len(cur.entries), "phase": "decode", "total_q": len(cur.entries)},
                })
        self._emit(emitted)

    def _drain(self, check: bool = True) -> None:
        """Read back whatever was launched ahead (used before the engine stops).  Without
        ``check`` (after a fault) the steps are waited for and their tokens thrown away."""
        while self._inflight is not None:
            cur, self._inflight = self._inflight, None
            if check:
                self._collect(cur)
                continue
            if cur.ready is not None:
                cur.ready.synchronize()
            with self._lock:
                for rr in cur.owners:
                    if rr.in_flight_after_done:
                        rr.in_flight_after_done = False
                        self._release(rr)
                    elif rr.state is not RequestState.DONE:
                        self._retire(rr, "cancelled")

    # ------------------------------------------------------------------ internals (lock held)

    def _pages(self, tokens: int) -> int:
        return -(-tokens // self.cache.page_size)

    def _admit(self) -> None:
        while self._waiting and len(self._live) < self.max_concurrent and self.cache.num_free_slots > 0:
            rr = self._waiting[0]
            need = self._pages(len(rr.feed) + 1)
            pool_pages = min(p.num_pages for p in self.cache.pools) if self.cache.pools else 0
            free_pages = min(p.num_free for p in self.cache.pools) if self.cache.pools else need
            if self.cache.pools and need > pool_pages:
                self._waiting.popleft()
                self._finish(rr, "cancelled")       # could never fit (reference :738-746)
                continue
            headroom = self.decode_headroom_blocks if self._live else 0
            if self.cache.pools and need + headroom > free_pages - self._reserved_pages():
                break                               # head of the line waits; nobody overtakes
            self._waiting.popleft()
            self.cache.add_request(rr.rid)
            rr.state = RequestState.PREFILLING
            rr.fed = 0
            rr.admitted_at = self._admissions
            self._admissions += 1
            self._live.append(rr)

    def _reserved_pages(self) -> int:
        """Pages that admitted, still prefilling requests will need for the rest of their prompts."""
        total = 0
        for rr in self._live:
            if rr.state is RequestState.PREFILLING:
                total += self._pages(len(rr.feed) + 1) - self._pages(rr.fed)
        return total

    def _plan(self) -> tuple[list[StepEntry], list[RunningRequest]]:
        """The next batch: decoders first, then prompt portions under the token budget;
        shrunk, and if need be with requests preempted, until its pages are there."""
        while True:
            decoders = [rr for rr in self._live if rr.state is RequestState.DECODING]
            prefillers = sorted((rr for rr in self._live if rr.state is RequestState.PREFILLING),
                                key=lambda r: r.admitted_at)
            budget = self.max_tokens_per_step
            plan: list[tuple[RunningRequest, int]] = []
            for rr in decoders:
                if budget <= 0:
                    break
                plan.append((rr, 1))
                budget -= 1
            for rr in prefillers:
                if budget <= 0:
                    break
                n = min(self.chunk_size, len(rr.feed) - rr.fed, budget)
                plan.append((rr, n))
                budget -= n
            if not plan:
                return [], []
            # shrink prompt portions, youngest first, until the pages are there
            while not self.cache.can_append([(rr.rid, n) for rr, n in plan]):
                idx = max((i for i, (rr, n) in enumerate(plan) if rr.state is RequestState.PREFILLING),
                          key=lambda i: plan[i][0].admitted_at, default=None)
                if idx is None:
                    break
                rr, n = plan[idx]
                held = self.cache.length(rr.rid)
                room = self._pages(held) * self.cache.page_size - held   # tokens that need no new page
                if 0 < room < n:
                    plan[idx] = (rr, room)
                else:
                    plan.pop(idx)
            if plan and self.cache.can_append([(rr.rid, n) for rr, n in plan]):
                break
            # even the decoding tokens do not fit: preempt the youngest live request
            victim = max(self._live, key=lambda r: r.admitted_at)
            if len(self._live) == 1:
                self._release(victim)
                self._live.remove(victim)
                self._finish(victim, "cancelled")   # cannot fit even alone
                return [], []
            self._preempt(victim)
        entries, owners = [], []
        for rr, n in plan:
            if rr.state is RequestState.DECODING:
                tokens, want = [rr.next_token], [0]
            else:
                tokens = rr.feed[rr.fed:rr.fed + n]
                want = [n - 1] if rr.fed + n == len(rr.feed) else []
            entries.append(StepEntry(rr.rid, tokens, want))
            owners.append(rr)
        return entries, owners

    def _preempt(self, rr: RunningRequest) -> None:
        self._release(rr)
        self._live.remove(rr)
        rr.feed = list(rr.prompt_ids) + list(rr.generated)
        # (a decoding request's pending token is the last of ``generated``, so it is in ``feed``)
        rr.fed = 0
        rr.next_token = None
        rr.state = RequestState.WAITING
        rr.preemptions += 1
        self.preemptions += 1
        self._waiting.appendleft(rr)

    def _release(self, rr: RunningRequest) -> None:
        if rr.rid in self.cache:
            self.cache.free_request(rr.rid)

    def _consume(self, rr: RunningRequest, token: int, still_in_flight: bool = False, emitted: list | None = None) -> None:
        """A sampled token: emit it, or finish the request (reference ``:847-860``).  With
        ``still_in_flight`` a step launched ahead holds the request: if it ends here, its
        pages stay until that step has been read.  The request's streaming callback is not
        called here (the lock is held) but noted in ``emitted`` for ``_emit``."""
        if token in self.eos_token_ids:
            self._retire(rr, "stop", still_in_flight)
            return
        rr.generated.append(token)
        rr.next_token = token
        self.tokens_generated += 1
        if rr.on_token is not None and emitted is not None:
            emitted.append((rr.on_token, token))
        held = self.cache.length(rr.rid) - (1 if still_in_flight else 0)   # without the token launched ahead
        if len(rr.generated) >= rr.request.max_tokens:
            self._retire(rr, "length", still_in_flight)
        elif self.max_positions is not None and held + 1 > self.max_positions:
            self._retire(rr, "length", still_in_flight)

    def _retire(self, rr: RunningRequest, reason: str, still_in_flight: bool = False) -> None:
        if still_in_flight:
            rr.in_flight_after_done = True
        else:
            self._release(rr)
        if rr in self._live:
            self._live.remove(rr)
        self._finish(rr, reason)

    def _finish(self, rr: RunningRequest, reason: str) -> None:
        rr.state = RequestState.DONE
        rr.finish_reason = reason
        rr.done.set()

    def _cancel(self, rr: RunningRequest) -> None:
        """Ask for cancellation; it takes effect at the start of the next engine step (or
        now, when no engine thread runs), never while a step is in flight."""
        with self._lock:
            if rr.state is RequestState.DONE:
                return
            rr.cancel_requested = True
            if self._thread is None:
                if rr in self._live:
                    held_ahead = self._inflight is not None and any(o is rr for o in self._inflight.owners)
                    self._retire(rr, "cancelled", still_in_flight=held_ahead)
                else:
                    try:
                        self._waiting.remove(rr)
                    except ValueError:
                        pass
                    self._finish(rr, "cancelled")
