"""The generation loop: batches of unequal prompts, stop tokens, early finishers.

Per request the order is the reference's (``src/generation/generator.cpp:617-803``):
check the prompt (non-empty, ids inside the vocabulary, room in the cache);
return the prompt unchanged if no new token is asked for or its last token is a
stop token; run the prompt; then repeat: logits of the last position, choose a
token, append it, stop if it is a stop token (it stays in the output) or the
budget is reached, else feed it back.  The last chosen token is never fed.

Beyond the reference, which runs one sequence (``seq_id`` 0), requests run in
batches that start together: their prompts in one step, then one token each per
step; a finished request leaves the batch at once and gives its slot and blocks
back; further batches follow until every request is served.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..sampling import SamplingParams
from .engine import StepEntry


class RequestError(ValueError):
    pass


@dataclass
class GenerationTimings:
    prefill_ms: float = 0.0
    prefill_tokens: int = 0
    decode_ms: float = 0.0
    decode_tokens: int = 0
    batches: int = 0

    @property
    def decode_tps(self) -> float:
        return 1000.0 * self.decode_tokens / self.decode_ms if self.decode_ms > 0 else 0.0


@dataclass
class GenerationOutput:
    sequences: List[List[int]]            # prompt followed by the generated ids, per request
    timings: GenerationTimings = field(default_factory=GenerationTimings)

    def generated(self, prompts: Sequence[Sequence[int]]) -> List[List[int]]:
        return [seq[len(p):] for seq, p in zip(self.sequences, prompts)]


def blocks_needed(tokens: int, block_size: int) -> int:
    return -(-tokens // block_size)


def plan_batches(needs: Sequence[int], free_blocks: int, free_slots: int) -> List[List[int]]:
    """Split requests (in order) into batches.  ``needs[i]`` is the number of
    cache blocks request ``i`` can grow to.  A batch takes requests while its
    blocks and slots last; a request that fits nowhere raises."""
    batches: List[List[int]] = []
    current: List[int] = []
    used = 0
    for index, need in enumerate(needs):
        if need > free_blocks:
            raise RequestError(f"request {index}: prompt plus max_new_tokens needs {need} cache blocks, "
                               f"the cache has {free_blocks}")
        if current and (used + need > free_blocks or len(current) >= free_slots):
            batches.append(current)
            current, used = [], 0
        current.append(index)
        used += need
    if current:
        batches.append(current)
    return batches


def validate_request(index: int, prompt: Sequence[int], max_new_tokens: int, vocab: int,
                     max_context: int = 0) -> None:
    """src/generation/generator.cpp:619-632: everything is checked before anything is touched."""
    if len(prompt) == 0:
        raise RequestError(f"request {index}: the prompt is empty")
    if max_new_tokens < 0:
        raise RequestError(f"request {index}: max_new_tokens must be nonnegative")
    for token in prompt:
        if not isinstance(token, int) or isinstance(token, bool) or not (0 <= token < vocab):
            raise RequestError(f"request {index}: prompt token {token!r} is outside the vocabulary of {vocab}")
    # the last chosen token is never fed, so a request reaches prompt + max_new_tokens - 1 positions in the cache
    if max_context and max_new_tokens > 0 and len(prompt) + max_new_tokens - 1 > max_context:
        raise RequestError(f"request {index}: a prompt of {len(prompt)} tokens plus {max_new_tokens} new ones "
                           f"exceeds the context limit of {max_context}")


def generate(engine, choose: Callable, prompts: Sequence[Sequence[int]], max_new_tokens,
             stop_ids: Sequence[int] = (), streams: Optional[Sequence[int]] = None,
             clock: Callable[[], float] = time.perf_counter, sync: Callable[[], None] = lambda: None
             ) -> GenerationOutput:
    """Serve ``prompts``.

    ``engine`` has ``open_sequence``, ``close_sequence``, ``step(entries)``, a
    ``cache`` with ``block_size``, free block counts and free slots,
    ``spec.vocab_size`` and (optionally) ``max_context``.  ``choose(logits, streams, counters)`` returns one token
    id per row as a list of ints.  ``max_new_tokens`` is one number or one per
    request.  ``streams[i]`` names request ``i``'s random stream (default ``i``).
    """
    count = len(prompts)
    budgets = [max_new_tokens] * count if isinstance(max_new_tokens, int) else list(max_new_tokens)
    if len(budgets) != count:
        raise RequestError("max_new_tokens must be one number or one per request")
    streams = list(range(count)) if streams is None else list(streams)
    stop = frozenset(int(s) for s in stop_ids)
    vocab = engine.spec.vocab_size
    max_context = getattr(engine, "max_context", 0)
    for index, prompt in enumerate(prompts):
        validate_request(index, prompt, budgets[index], vocab, max_context)
    sequences = [list(p) for p in prompts]
    # src/generation/generator.cpp:627: nothing to do for these requests
    active = [i for i in range(count) if budgets[i] > 0 and sequences[i][-1] not in stop]
    block_size = engine.cache.block_size
    free_blocks = min(engine.cache.free_blocks()) if engine.cache.free_blocks() else 10 ** 9
    needs = [blocks_needed(len(prompts[i]) + budgets[i], block_size) for i in active]
    timings = GenerationTimings()
    for batch in plan_batches(needs, free_blocks, engine.cache.slots.free_count):
        members = [active[j] for j in batch]
        _run_batch(engine, choose, members, sequences, prompts, budgets, stop, streams, timings, clock, sync)
        timings.batches += 1
    return GenerationOutput(sequences, timings)


def _take(engine, members, tokens, slots, sequences, prompts, budgets, stop):
    """Append each member's new token; a member whose token is a stop token or whose budget is reached leaves the
    batch at once (its slot and blocks go back).  Returns the members that go on."""
    still = []
    for i, token in zip(members, tokens):
        sequences[i].append(int(token))
        produced = len(sequences[i]) - len(prompts[i])
        if int(token) in stop or produced >= budgets[i]:
            engine.close_sequence(slots.pop(i))
        else:
            still.append(i)
    return still


def _decode_in_turn(engine, choose, live, chosen, slots, sequences, prompts, budgets, stop, streams, timings):
    """Step, choose, read the tokens, step again: the host knows every token before it feeds it."""
    while True:
        live = _take(engine, live, chosen, slots, sequences, prompts, budgets, stop)
        if not live:
            return
        logits = engine.step([StepEntry(slots[i], [sequences[i][-1]], [0]) for i in live])
        chosen = choose(logits, [streams[i] for i in live], [len(sequences[i]) - len(prompts[i]) for i in live])
        timings.decode_tokens += len(live)


def _decode_ahead(engine, chooser, live, chosen, slots, sequences, prompts, budgets, stop, streams, timings):
    """The same results with the host one step behind the device: while it reads the tokens that a step chose,
    the next step, fed with those tokens where they lie on the device, is already running.  A step is launched
    ahead only for the very members of the step before it and only if none of them can reach its budget with
    the token still unread; a member that turns out to have hit a stop token has then run one step in vain
    (its row is dropped, its slot was still its own), and the loop falls back in step with the host."""
    produced = lambda i: len(sequences[i]) - len(prompts[i])
    live = _take(engine, live, chosen, slots, sequences, prompts, budgets, stop)
    flying = None                                        # (members, handle): a step in flight whose tokens are unread
    while live or flying:
        if flying is None:
            logits = engine.step([StepEntry(slots[i], [sequences[i][-1]], [0]) for i in live])
            flying = (list(live), chooser.launch(logits, [streams[i] for i in live], [produced(i) for i in live]))
        members, handle = flying
        following = None
        if all(produced(i) + 1 < budgets[i] for i in members):
            logits = engine.step_ahead([slots[i] for i in members], chooser.tokens_device(handle))
            following = chooser.launch(logits, [streams[i] for i in members], [produced(i) + 1 for i in members])
        tokens = chooser.result(handle)
        timings.decode_tokens += len(members)
        live = _take(engine, members, tokens, slots, sequences, prompts, budgets, stop)
        if following is None:
            flying = None
        elif live == members:
            flying = (members, following)
        else:                                            # somebody stopped: the step ahead ran a row for it in vain
            tokens = chooser.result(following)
            going = set(live)
            pairs = [(i, token) for i, token in zip(members, tokens) if i in going]
            timings.decode_tokens += len(pairs)
            live = _take(engine, [i for i, _ in pairs], [token for _, token in pairs], slots, sequences, prompts,
                         budgets, stop)
            flying = None


def _run_batch(engine, choose, members, sequences, prompts, budgets, stop, streams, timings, clock, sync):
    slots = {}
    try:
        for i in members:
            slots[i] = engine.open_sequence()
        live = list(members)
        sync()
        start = clock()
        logits = engine.step([StepEntry(slots[i], prompts[i], [len(prompts[i]) - 1]) for i in live])
        chosen = choose(logits, [streams[i] for i in live], [0] * len(live))
        sync()
        timings.prefill_ms += 1000.0 * (clock() - start)
        timings.prefill_tokens += sum(len(prompts[i]) for i in live)
        start = clock()
        ahead = hasattr(choose, "launch") and getattr(engine, "can_step_ahead", False)
        (_decode_ahead if ahead else _decode_in_turn)(engine, choose, live, chosen, slots, sequences, prompts, budgets,
                                                       stop, streams, timings)
        sync()
        timings.decode_ms += 1000.0 * (clock() - start)
    finally:
        for slot in slots.values():                              # on an error, give everything back
            engine.close_sequence(slot)
