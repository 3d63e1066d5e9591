"""The allocation-free split-KV attention entry point (csrc/attention_noalloc.h), called through its
exported C symbol, against the ordinary entry point that takes a scratch buffer from its caller.

Some users of the library cannot allocate device memory where they call it (inside a graph capture, in a
real-time loop, in a process whose memory was handed out at start-up); for them the scratch lives in a
fixed array inside the library.  The test makes two calls in a row of different sizes, so that the second
finds the first one's leftovers in that array, and wants the same bits as the ordinary entry point both
times.  It is collected last: a run that stops at the first failure has then run everything else."""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE = -27
CAPACITY = 1 << 20


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _libs():
    from kappai_b200.ops.build import load_library
    new, old = load_library("attention_noalloc"), load_library("attention_decode")
    new.kp_attention_split_noalloc_need.restype = ctypes.c_longlong
    new.kp_attention_split_noalloc_strerror.restype = ctypes.c_char_p
    return new, old


def _case(rng, seq_lens, H, G, hd, page, dtype):
    """Scattered pages, one decode row per request."""
    blocks = [-(-L // page) for L in seq_lens]
    n_pages = sum(blocks) + 2
    perm = rng.permutation(n_pages)
    cache = torch.as_tensor(rng.standard_normal((n_pages, 2, G, page, hd)).astype(np.float32)).to(dtype).cuda()
    bt = np.full((len(seq_lens), max(blocks)), -1, np.int32)
    o = 0
    for i, nb in enumerate(blocks):
        bt[i, :nb] = perm[o:o + nb]
        o += nb
    n = len(seq_lens)
    q = torch.as_tensor(rng.standard_normal((n, H * hd)).astype(np.float32)).to(dtype).cuda()
    i32 = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int32)).cuda()
    return q, cache, i32(bt), i32(list(range(n))), i32([L - 1 for L in seq_lens])


def _both(new, old, q, cache, bt, row_seg, pos, H, G, hd, page, window, dtype):
    n = q.shape[0]
    n_chunks = -(-(int(pos.max().item()) + 1) // 256)
    code = 0 if dtype == torch.float32 else 1
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    scale = ctypes.c_float(1.0 / math.sqrt(hd))
    out_new = torch.full((n, H * hd), float("nan"), dtype=dtype, device="cuda")
    st = new.kp_attention_split_noalloc(_ptr(q), q.stride(0), _ptr(cache), _ptr(bt), bt.shape[1], _ptr(row_seg), _ptr(pos),
                                        _ptr(out_new), out_new.stride(0), n_chunks, scale, window, page, n, H, G, hd,
                                        code, stream)
    assert st == 0, new.kp_attention_split_noalloc_strerror(st)
    need = new.kp_attention_split_noalloc_need(n, H, hd, n_chunks)
    scratch = torch.full((need,), float("nan"), device="cuda")           # the ordinary way: the caller's buffer
    out_old = torch.full((n, H * hd), float("nan"), dtype=dtype, device="cuda")
    st = old.kp_attention_split(_ptr(q), q.stride(0), _ptr(cache), _ptr(bt), bt.shape[1], _ptr(row_seg), _ptr(pos),
                                _ptr(out_old), out_old.stride(0), _ptr(scratch), n_chunks, scale, window, page, n, H, G,
                                hd, code, stream)
    assert st == 0
    torch.cuda.synchronize()
    return out_new, out_old


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_calls_in_a_row_match_the_ordinary_entry_point(dtype):
    new, old = _libs()
    rng = np.random.default_rng(70)
    # first a large call (fills much of the array), then a smaller one with other sizes and a window
    for seq_lens, H, G, hd, page, window in (([700, 300, 1025, 64], 8, 2, 64, 64, 0), ([257, 90], 6, 3, 48, 16, 100)):
        q, cache, bt, row_seg, pos = _case(rng, seq_lens, H, G, hd, page, dtype)
        got, want = _both(new, old, q, cache, bt, row_seg, pos, H, G, hd, page, window, dtype)
        assert not torch.isnan(got.float()).any()
        tol = 2e-5 if dtype == torch.float32 else 1.2e-2            # the tolerances of the kernel tests
        assert (got.float() - want.float()).abs().max().item() <= tol
        assert torch.equal(got, want)                                # the same kernels: in fact the same bits


def test_a_call_beyond_the_array_is_refused():
    new, _ = _libs()
    n, H, hd, n_chunks = 64, 32, 64, 16                              # 64*32*16*66 floats: twice the array
    assert new.kp_attention_split_noalloc_need(n, H, hd, n_chunks) > CAPACITY
    q = torch.zeros((n, H * hd), device="cuda")
    out = torch.full_like(q, 7.0)
    z = torch.zeros(n, dtype=torch.int32, device="cuda")
    st = new.kp_attention_split_noalloc(_ptr(q), q.stride(0), _ptr(q), _ptr(z), 1, _ptr(z), _ptr(z), _ptr(out),
                                        out.stride(0), n_chunks, ctypes.c_float(1.0), 0, 64, n, H, 8, hd, 0,
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == TOO_LARGE
    assert b"scratch" in new.kp_attention_split_noalloc_strerror(st)
    torch.cuda.synchronize()
    assert (out == 7.0).all()                                        # nothing was launched
