"""A step that fails must fail: nothing of it is kept, its requests end with an error, and the slot
serves the next request as if nothing had happened.  Every failure here is made on the host: a NaN
written into a weight row, or a fault word of the engine's status buffer set from the test.  No
kernel is made to wait, trap or read a bad address."""
import numpy as np
import pytest
import torch
from conftest import TINY
from helpers import TOL, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


def build(folder, dtype="float32", **kw):
    from safetyraise_lmengine_b200 import Engine
    kw.setdefault("num_pages", 24)
    kw.setdefault("page_size", 4)
    return Engine.from_folder(folder, dtype=dtype, max_requests=4, max_batch_tokens=256, **kw)


def state_of(eng, slot):
    return eng.cache.length(slot), eng.cache.free_pages(), eng.cache.audit()


@pytest.mark.parametrize("word", [0, 1, 2, 3])
def test_raised_fault_word_fails_the_step_and_keeps_nothing(folder_a, word):
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.errors import StepFailed
    eng = build(folder_a)
    rng = np.random.default_rng(word)
    toks = random_tokens(rng, 19, TINY["A"][0]["vocab_size"])
    ref = plain_logits(folder_a, toks)
    s = eng.open_request()
    eng.step([StepEntry(s, toks[:7], [6])])
    before = state_of(eng, s)
    eng.status[word] = 5                                     # the host stands in for the kernel that raises it
    with pytest.raises(StepFailed) as err:
        eng.step([StepEntry(s, toks[7:16], [8])])
    assert err.value.words[word] == 5 and sum(1 for w in err.value.words if w) == 1
    assert state_of(eng, s) == before == (7, before[1], 0)
    assert eng.read_faults() == [0] * 8                      # read and cleared: the next step starts clean
    got = eng.step([StepEntry(s, toks[7:], list(range(12)))]).cpu().numpy()
    assert np.abs(got - ref[7:]).max() <= TOL["float32"] * np.abs(ref).max()
    eng.close_request(s)
    assert eng.cache.free_pages() == 24 and eng.cache.audit() == 0 and eng.steps_failed == 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_nan_in_an_embedding_row_fails_only_steps_that_read_it(folder_b, dtype):
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.errors import StepFailed
    from safetyraise_lmengine_b200.parts.base import FAULT_ACTIVATION
    eng = build(folder_b, dtype)
    vocab = TINY["B"][0]["vocab_size"]
    rng = np.random.default_rng(4)
    clean = [t for t in random_tokens(rng, 40, vocab) if t != 11][:30]
    ref = plain_logits(folder_b, clean)
    eng.model.embed[11].fill_(float("nan"))                  # untied: the output head stays whole
    s = eng.open_request()
    eng.step([StepEntry(s, clean[:10], [])])
    free = eng.cache.free_pages()
    with pytest.raises(StepFailed) as err:                   # a portion with no wanted place fails all the same
        eng.step([StepEntry(s, [3, 11, 5, 8, 2, 2, 9], [])])
    assert err.value.words[FAULT_ACTIVATION] == 1
    assert (eng.cache.length(s), eng.cache.free_pages(), eng.cache.audit()) == (10, free, 0)
    with pytest.raises(StepFailed):                          # a decoded token beside another request's portion
        s2 = eng.open_request()
        eng.step([StepEntry(s, [11], [0]), StepEntry(s2, clean[:5], [4])])
    assert eng.cache.length(s) == 10 and eng.cache.length(s2) == 0
    eng.close_request(s2)
    got = eng.step([StepEntry(s, clean[10:], list(range(20)))]).cpu().numpy()
    assert np.abs(got - ref[10:]).max() <= TOL[dtype] * np.abs(ref).max()
    eng.close_request(s)
    assert eng.cache.free_pages() == 24 and eng.cache.audit() == 0


def test_nan_in_the_output_head_is_a_fault_of_the_logits(folder_b):
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.errors import StepFailed
    from safetyraise_lmengine_b200.parts.base import FAULT_ACTIVATION, FAULT_LOGITS
    eng = build(folder_b)
    eng.model.head.weight[17, 3] = float("inf")
    s = eng.open_request()
    eng.step([StepEntry(s, [1, 2, 3], [])])                  # nothing wanted: the head does not run
    with pytest.raises(StepFailed) as err:
        eng.step([StepEntry(s, [4, 5], [1])])
    assert err.value.words[FAULT_LOGITS] == 1 and err.value.words[FAULT_ACTIVATION] == 0
    assert eng.cache.length(s) == 3 and eng.cache.audit() == 0


def test_a_slot_that_changed_hands_is_refused(folder_a):
    """src/model/native.rs:259-261: a state that belongs to another owner is an error."""
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.errors import ShapeError
    eng = build(folder_a)
    s = eng.open_request()
    mine = eng.generation(s)
    eng.step([StepEntry(s, [1, 2, 3], [2], generation=mine)])
    eng.close_request(s)
    s2 = eng.open_request()                                  # the slot freed last is handed out next
    assert s2 == s and eng.generation(s2) == mine + 1
    with pytest.raises(ShapeError, match="another request"):
        eng.step([StepEntry(s, [4], [0], generation=mine)])
    assert eng.cache.length(s2) == 0 and eng.cache.audit() == 0
    eng.step([StepEntry(s2, [4], [0], generation=eng.generation(s2))])


def llm_for(folder, dtype="float32", **kw):
    from safetyraise_lmengine_b200 import LLM
    kw.setdefault("num_pages", 40)
    return LLM.from_folder(folder, dtype=dtype, page_size=4, max_active=4, queue_capacity=8,
                           max_batch_tokens=256, prefill_chunk=16, max_context=128, **kw)


def plain_greedy(folder, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(plain_logits(folder, toks)[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("plan_ahead, launch_ahead", [(True, True), (True, False), (False, False)])
def test_generation_ends_a_failed_steps_requests_with_error(folder_b, plan_ahead, launch_ahead):
    """The scheduler's side (src/engine/scheduler.rs:882-895): the requests of the failed step end
    with ``error``, their pages and slots come back, and the engine goes on serving.  With a step
    queued ahead, the step that was already on the device when the weight broke is a sound one: its
    tokens are published, and the step queued behind the failed one is taken back."""
    from safetyraise_lmengine_b200 import GenerationRequest, SamplingParams
    llm = llm_for(folder_b, plan_ahead=plan_ahead, launch_ahead=launch_ahead)
    eng = llm.engine
    vocab = TINY["B"][0]["vocab_size"]
    rng = np.random.default_rng(2)
    prompts = [random_tokens(rng, n, vocab) for n in (9, 21)]
    greedy = SamplingParams(temperature=0.0, max_new_tokens=12)
    down = eng.model.blocks[1].feed_forward.down.weight
    kept = down[5].clone()
    ids = [llm.submit(GenerationRequest(p, SamplingParams(**vars(greedy)))) for p in prompts]
    seen = []
    for _ in range(6):                                       # prompts are in, decoding has begun
        llm.step(lambda rid, tok, i: seen.append((rid, tok)))
    assert len(seen) >= 4
    torch.cuda.synchronize()                                 # (a step queued ahead has run with sound weights)
    down[5].fill_(float("nan"))                              # the failure, made on the host
    published = len(seen)
    llm.run_until_idle(lambda rid, tok, i: seen.append((rid, tok)))
    # no token of a failed step is published; the sound step that was on the device already publishes its two
    assert len(seen) == published + (2 if launch_ahead else 0)
    for rid, p in zip(ids, prompts):
        got = [tok for r, tok in seen if r == rid]
        assert got == plain_greedy(folder_b, p, 12)[:len(got)]
    assert llm.steps_dropped == (1 if launch_ahead else 0)
    for rid in ids:
        res = llm.take_result(rid)
        assert res.finish_reason == "error" and "non-finite" in res.error
    assert eng.cache.free_pages() == 40 and eng.cache.audit() == 0 and llm.metrics()["failed"] == 2
    assert eng.steps_failed == 1
    down[5].copy_(kept)                                      # repaired: the same slots serve new requests
    out = llm.generate(prompts, greedy)
    for p, res in zip(prompts, out):
        assert res.finish_reason == "length" and res.tokens == plain_greedy(folder_b, p, 12)
    assert eng.cache.free_pages() == 40 and eng.cache.audit() == 0


def test_generation_reads_a_fault_word_raised_during_a_prompt_portion(folder_a):
    """A step with no row to sample still reads the fault words before anything is kept."""
    from safetyraise_lmengine_b200 import GenerationRequest, SamplingParams
    llm = llm_for(folder_a)
    rid = llm.submit(GenerationRequest(list(range(40)), SamplingParams(temperature=0.0, max_new_tokens=4)))
    assert llm.step()                                        # the first 16 tokens of the prompt
    llm.engine.status[0] = 1                                 # as if a bounded wait had run out
    assert llm.step()                                        # the second portion: nothing is sampled
    res = llm.take_result(rid)
    assert res is not None and res.finish_reason == "error" and "bounded wait" in res.error
    assert llm.engine.cache.free_pages() == 40 and llm.engine.cache.audit() == 0
    assert not llm.step()


def test_a_wait_that_runs_out_raises_the_word_and_fails_the_step(folder_a):
    """A bounded wait that really runs out on the device: the pipelines' own wait, on a barrier that nobody
    arrives at, with a limit of a million cycles.  The kernel raises the engine's word, ends normally, the
    step that was on the device with it keeps nothing, and the context goes on working."""
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.errors import ShapeError, StepFailed
    from safetyraise_lmengine_b200.kernels import ops
    eng = build(folder_a)
    rng = np.random.default_rng(9)
    toks = random_tokens(rng, 19, TINY["A"][0]["vocab_size"])
    ref = plain_logits(folder_a, toks)
    s = eng.open_request()
    eng.step([StepEntry(s, toks[:7], [6])])
    before = state_of(eng, s)
    t0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0[0].record()
    ops.wait_probe(eng.status[:1], limit_cycles=1_000_000, code=77)       # the word a pipeline's wait raises
    t0[1].record()
    with pytest.raises(StepFailed, match="bounded wait") as err:
        eng.step([StepEntry(s, toks[7:16], [8])])
    assert err.value.words[0] == 77 and sum(1 for w in err.value.words if w) == 1
    assert 0.1 < t0[0].elapsed_time(t0[1]) < 50.0            # it waited for its limit (about half a millisecond)
    assert state_of(eng, s) == before
    assert eng.read_faults() == [0] * 8
    got = eng.step([StepEntry(s, toks[7:], list(range(12)))]).cpu().numpy()
    assert np.abs(got - ref[7:]).max() <= TOL["float32"] * np.abs(ref).max()
    eng.close_request(s)
    assert eng.cache.free_pages() == 24 and eng.cache.audit() == 0 and eng.steps_failed == 1
    # the library's own flag, read and cleared by gemm_error_flag
    ops.bind_error_flag(None)
    ops.wait_probe(ops._gemm_state(eng.status.device)[1], limit_cycles=200_000, code=5)
    assert ops.gemm_error_flag(eng.status.device) == 5 and ops.gemm_error_flag(eng.status.device) == 0
    with pytest.raises(ShapeError):
        ops.wait_probe(eng.status[:1], limit_cycles=3_000_000_000)        # beyond a second: refused
