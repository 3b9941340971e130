"""Failures made on the host, a wait that is made to run out within its limit, buffers poisoned
before use, and recorded steps enqueued without synchronising: what the engine does when
something goes wrong, and that nothing reads what nobody wrote. No test here faults, traps or
hangs the device."""
import numpy as np
import pytest
import torch

from helpers import TINY, TOL, TraceBuilder, compare_trace, embed_scale_for, make_model_dir, plain_logits, random_tokens, run_trace_engine

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders():
    return {name: make_model_dir(raw, seed) for name, (raw, seed) in TINY.items()}


def _engine(folder, dtype="bfloat16", **kw):
    from kapel_b200.engine import Engine

    kw.setdefault("max_tokens", 512)
    kw.setdefault("max_sequences", 8)
    return Engine.from_dir(folder, dtype=dtype, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_recorded_steps_enqueued_without_a_sync_equal_the_same_steps_synchronised(folders, dtype):
    """Sixteen decode passes of three requests through `Engine.step`, nothing waited for in between
    (the logits cloned on the stream), against the same passes with a synchronise after each: bit
    for bit. The host runs far ahead of the device here, so a staging buffer rewritten before its
    copy has run would feed a pass another pass's positions and block tables. A long first pass
    (a prompt portion) keeps the device busy while the host enqueues."""
    from kapel_b200.engine import StepEntry

    raw, _ = TINY["B"]
    rng = np.random.default_rng(41)
    prompts = {f"r{i}": random_tokens(rng, n, raw["vocab_size"]) for i, n in enumerate([70, 33, 5])}
    feed = {r: random_tokens(rng, 16, raw["vocab_size"]) for r in prompts}
    outs = []
    for sync in (True, False):
        engine = _engine(folders["B"], dtype)
        engine.step([StepEntry(r, p, []) for r, p in prompts.items()])
        engine.step([StepEntry(r, [feed[r][0]], [0]) for r in prompts])        # the recording is made here
        torch.cuda.synchronize()
        busy = StepEntry("busy", random_tokens(rng, 200, raw["vocab_size"]), [])
        engine.step([busy])                                                      # the device has work; the host goes on
        kept = []
        for i in range(1, 16):
            logits = engine.step([StepEntry(r, [feed[r][i]], [0]) for r in prompts])
            kept.append(logits.clone())
            if sync:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        assert engine.recorded_passes >= 15
        outs.append(torch.stack(kept).cpu().numpy())
    assert np.isfinite(outs[0]).all()
    assert np.array_equal(outs[0], outs[1])


def test_a_failed_recording_loses_only_the_recording(folders):
    """The capture of a decode pass is made to fail (on the host, inside the capture): the pass
    still returns its logits, eagerly, equal to a recorded pass's bit for bit; the size is
    remembered as unrecordable, not tried again for 256 passes, then recorded; requests go on."""
    from kapel_b200.engine import StepEntry
    from kapel_b200.engine.graph import RETRY_AFTER

    raw, _ = TINY["A"]
    rng = np.random.default_rng(42)
    prompt = random_tokens(rng, 20, raw["vocab_size"])
    feed = random_tokens(rng, 8, raw["vocab_size"])
    want = []
    good = _engine(folders["A"])
    good.step([StepEntry("a", prompt, [])])
    for t in feed:
        want.append(good.step([StepEntry("a", [t], [0])]).float().cpu().numpy())
    assert good.recorded_passes == len(feed)

    engine = _engine(folders["A"])
    engine.graphs.fail_next_captures = 1
    engine.step([StepEntry("a", prompt, [])])
    got = [engine.step([StepEntry("a", [t], [0])]).float().cpu().numpy() for t in feed]
    assert engine.graphs.failed_captures == 1 and "injected" in engine.graphs.last_capture_error
    assert engine.recorded_passes == 0 and len(engine.graphs.unrecordable) == 1      # eager all the way, one attempt only
    for g, w in zip(got, want):
        assert np.array_equal(g, w)
    engine.graphs.passes += RETRY_AFTER                                              # as if 256 passes had gone by
    again = engine.step([StepEntry("a", [feed[0]], [0])])
    assert engine.recorded_passes == 1 and not engine.graphs.unrecordable and torch.isfinite(again).all()
    engine.end("a")
    assert engine.cache.free_pages() == engine.cache.total_pages()


def test_a_failed_recording_under_the_scheduler_ends_nobody(folders):
    import kapel_b200
    from kapel_b200.engine.scheduler import Request

    raw, _ = TINY["A"]
    rng = np.random.default_rng(43)
    prompts = [random_tokens(rng, n, raw["vocab_size"]) for n in (12, 30)]
    model = kapel_b200.Model(str(folders["A"]), dtype="f32", max_tokens_cached=512, max_sequences=4)
    want = [model.generate(p, max_tokens=12) for p in prompts]
    other = kapel_b200.Model(str(folders["A"]), dtype="f32", max_tokens_cached=512, max_sequences=4)
    other.engine.graphs.fail_next_captures = 2
    sched = other.scheduler(max_pass_tokens=64)
    ids = [sched.add(Request(p, max_tokens=12)) for p in prompts]
    out = {r: [] for r in ids}
    while sched.has_work():
        for ev in sched.step():
            assert ev.finish != "error", ev.error
            if ev.token is not None:
                out[ev.id].append(ev.token)
    assert [out[r] for r in ids] == want
    assert other.engine.graphs.failed_captures >= 1


def test_an_allocation_that_fails_inside_a_step_leaves_the_engine_whole(folders):
    """The fifth buffer a step asks for is refused as if the device were full (injected on the host):
    the step raises, its pages go back, a request that came with it is gone again, lengths have not
    moved; the same step then runs and gives the plain logits. Under the scheduler the failed pass
    ends the running requests and every page is free."""
    import kapel_b200
    from kapel_b200 import kernels as K
    from kapel_b200.engine import StepEntry
    from kapel_b200.engine.scheduler import Request

    raw, _ = TINY["A"]
    rng = np.random.default_rng(44)
    toks = random_tokens(rng, 40, raw["vocab_size"])
    engine = _engine(folders["A"], "float32")
    engine.step([StepEntry("old", toks[:10], [])])
    free = engine.cache.free_pages()
    K.fail_allocation_in(5)
    try:
        with pytest.raises(torch.OutOfMemoryError, match="injected"):
            engine.step([StepEntry("old", toks[10:20], [9]), StepEntry("new", toks[:7], [6])])
    finally:
        K.fail_allocation_in(0)
    assert engine.cache.free_pages() == free and engine.cache.length("old") == 10 and "new" not in engine.cache
    engine.cache.check()
    got = engine.step([StepEntry("old", toks[10:20], [9]), StepEntry("new", toks[:7], [6])]).cpu().numpy()
    plain = plain_logits(folders["A"], toks[:20], embed_scale=embed_scale_for(raw, "float32"))
    assert np.abs(got[0] - plain[19]).max() / np.abs(plain[19]).max() <= TOL["float32"]
    assert np.abs(got[1] - plain[6]).max() / np.abs(plain[6]).max() <= TOL["float32"]

    model = kapel_b200.Model(str(folders["A"]), dtype="f32", max_tokens_cached=512, max_sequences=4)
    model.engine.graphs = None              # eager passes: a failure while recording would only lose the recording
    sched = model.scheduler()
    ids = [sched.add(Request(toks[:9], max_tokens=20)), sched.add(Request(toks[9:30], max_tokens=20))]
    sched.step()
    K.fail_allocation_in(3)
    try:
        events = sched.step()
    finally:
        K.fail_allocation_in(0)
    assert sorted(e.id for e in events) == ids and all(e.finish == "error" and "injected" in e.error for e in events)
    assert not sched.has_work() and model.engine.cache.free_pages() == model.engine.cache.total_pages()
    assert model.generate(toks[:9], max_tokens=4)                       # and the model still generates


def test_a_wait_that_runs_out_raises_its_flag_and_the_device_goes_on(folders):
    """One small block waits, with the products' own bounded wait and a limit of about a
    millisecond, on a barrier at which nothing ever arrives. The wait gives up, the kernel returns,
    `check_async_errors` reports it once, and the kernels after it run as ever."""
    from kapel_b200 import kernels as K
    from kapel_b200.engine import StepEntry

    K.check_async_errors()                                  # nothing pending from earlier tests
    K.wait_probe(2_000_000)
    with pytest.raises(K.KernelError, match="gave up after its time limit.*tcgen05 product"):
        K.check_async_errors()
    K.check_async_errors()                                  # the flag was cleared by the report
    with pytest.raises(K.KernelError, match="wait_probe"):
        K.wait_probe(10 ** 9)                               # a limit beyond the launcher's bound is refused, nothing launched
    raw, _ = TINY["A"]
    toks = random_tokens(np.random.default_rng(45), 30, raw["vocab_size"])
    engine = _engine(folders["A"])
    got = engine.step([StepEntry("a", toks, [29])]).float().cpu().numpy()
    plain = plain_logits(folders["A"], toks, embed_scale=embed_scale_for(raw, "bfloat16"))
    assert np.abs(got[0] - plain[29]).max() / np.abs(plain[29]).max() <= TOL["bfloat16"]
    K.check_async_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_the_four_cuts_with_every_fresh_buffer_poisoned(folders, name, dtype):
    """With every buffer a kernel is about to write filled with NaN first (outputs, scratch,
    split-K partial sums), the four ways of cutting the work still give the plain logits: no
    kernel reads what nobody wrote or leaves part of its output unwritten. Recorded decode
    passes run with the poisoning kernels inside the recording."""
    import test_gpu_engine as E
    from kapel_b200 import kernels as K

    K.set_poison(True)
    try:
        E.test_whole(folders, name, dtype)
        E.test_last_32_one_by_one(folders, name, dtype)
        E.test_portions_of_changing_size(folders, name, dtype)
        E.test_mixed_with_pages_used_again(folders, name, dtype)
    finally:
        K.set_poison(False)
