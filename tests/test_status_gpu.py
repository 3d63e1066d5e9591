"""A kernel that gives up a bounded wait is seen by the host: the status word travels with the step's tokens,
the step's requests end with ``compute_failed`` and give back what they hold, and the engine goes on
(the reference ends a session whose compute failed: src/context.c:1580-1592,1676-1680,
src/test/test_orchestration.c:684).  Nothing here faults or hangs: the failure is either a word the host
sets, or one stage of a product's ring that is left unfilled so that a wait of a millisecond runs out."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def engine(model_dir, **kw):
    from kappai_b200 import Engine, EngineArgs
    args = dict(model=model_dir, dtype="bfloat16", max_batch=4, max_step_tokens=32, page_size=16, kv_tokens=1024)
    args.update(kw)
    return Engine(EngineArgs(**args))


@pytest.mark.parametrize("look_ahead", [False, True])
def test_a_failed_step_ends_its_requests_and_the_engine_goes_on(look_ahead, model_dirs):
    from kappai_b200 import SamplingParams
    from kappai_b200.engine.runner import EngineError
    eng = engine(model_dirs["B"], look_ahead=look_ahead)
    rng = np.random.default_rng(5)
    sp = SamplingParams(temperature=0.0, n_predict=20)
    a = eng.add_request(rng.integers(0, 512, 12).tolist(), sp)
    b = eng.add_request(rng.integers(0, 512, 20).tolist(), sp)
    for _ in range(6):
        eng.step()
    assert len(eng.requests[a].output) >= 3
    eng.status.injected.fill_(1)                       # stands for a kernel's status word that rose
    with pytest.raises(EngineError, match="bounded wait gave up.*injected.*compute_failed"):
        eng.step()
        eng.step()                                     # (a step launched ahead was already under way: the next one sees it)
    assert eng.finish_reason(a) == eng.finish_reason(b) == "compute_failed"
    assert not eng.has_work()
    eng.runner.cache.check()
    assert eng.runner.cache.slots.n_free == 4 and all(p.n_free == p.n_pages for p in eng.runner.cache.pools.values())
    # the word is cleared and the engine serves the next request as if nothing had been
    prompt = rng.integers(0, 512, 9).tolist()
    got = eng.generate([prompt], sp)[0]
    want = engine(model_dirs["B"]).generate([prompt], sp)[0]
    assert got == want and len(got) == 20


def test_a_wait_that_runs_out_returns_and_sets_the_status_word():
    """The weight-streaming product built with its test hooks: CTA 0's producer leaves one stage of its ring
    unfilled and the waits give up after a millisecond.  The kernel returns, the status word reads 1 and then 0,
    the step's gathered word shows it, and the next ordinary launch is right."""
    from kappai_b200.ops import kernels as Kn
    from kappai_b200.ops.build import load_library
    lib = load_library("gemm_stream", variant="hooks", extra_flags=["-DKP_TEST_HOOKS"])
    M, N, Kd = 8, 2048, 1024
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn((M, Kd), device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn((N, Kd), device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    ref = a.float() @ w.float().t()

    def run():
        out = torch.full((M, N), float("nan"), device="cuda")
        st = lib.kp_gemm_stream(Kn._ptr(a), Kd, Kn._ptr(w), Kd, None, Kn._ptr(out), N, M, N, Kd, Kn.EPI_STORE_F32,
                                Kn._stream())
        assert st == 0
        torch.cuda.synchronize()
        return out

    fn = lib.kp_stream_status_address
    fn.restype = ctypes.c_void_p
    word = torch.zeros(1, dtype=torch.int32, device="cuda")
    addrs = torch.tensor([fn()], dtype=torch.int64).cuda()
    gather = lambda: (load_library("rowwise").kp_gather_status(Kn._ptr(addrs), 1, Kn._ptr(word), Kn._stream()),
                      int(word.item()))[1]

    assert torch.allclose(run(), ref, atol=2e-2, rtol=2e-2) and lib.kp_stream_status() == 0 and gather() == 0
    assert lib.kp_gemm_stream_test_fault(1, ctypes.c_ulonglong(1_000_000)) == 0     # its second stage unfilled, waits of 1 ms
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    bad = run()
    t1.record(); torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 500.0                                              # it gave up, it did not hang
    assert gather() == 1                                                            # what the engine would see
    assert lib.kp_stream_status() == 1 and lib.kp_stream_status() == 0               # read and cleared
    del bad                                              # (not to be trusted; whatever lay in the unfilled stage went into it)
    assert lib.kp_gemm_stream_test_fault(-1, ctypes.c_ulonglong(0)) == 0
    assert torch.allclose(run(), ref, atol=2e-2, rtol=2e-2) and lib.kp_stream_status() == 0 and gather() == 0


def test_replay_ends_with_an_error_when_a_status_word_is_set(model_dirs):
    from kappai_b200 import ModelRunner, StepEntry
    from kappai_b200.engine.runner import EngineError
    from kappai_b200.ops import kernels as Kn
    r = ModelRunner(model_dirs["A"], dtype="bfloat16", max_tokens=256, page_size=16)
    r.step([StepEntry("a", [1, 2, 3], [2])])
    r.check_status()
    real = Kn.read_status
    try:
        Kn.read_status = lambda: {"gemm_tc": 1, "gemm_stream": 0}
        with pytest.raises(EngineError, match="gemm_tc"):
            r.check_status()
    finally:
        Kn.read_status = real
