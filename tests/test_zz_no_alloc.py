"""-m gpu, collected last: mb_sample_noalloc, the one entry point of the kernel libraries that allocates nothing.

Some programs that call these kernels cannot allocate device memory: they gave the GPU's memory to their own pools at
start-up, or they must not take the driver's allocation lock in their loop, or they run under another program's memory
manager.  For them the sampling kernel's scratch lives in a fixed 2 MiB array inside the library.  This test calls
the exported C symbol directly (ctypes, raw pointers), twice in a row so that the second call finds the first one's
scratch, and checks each result against the ordinary entry point, which takes its scratch from the caller: the tokens
must be equal, as everywhere in the sampling tests.  It also checks that sizes beyond the fixed array are refused with
words, and that the device's free memory (as the driver reports it, whoever allocates) does not change over a call
once the library's image, with its fixed array, has been loaded by the first call.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def library():
    from mashbox_b200.ops.build import load_library
    lib = load_library("sampling_noalloc")
    lib.mb_sample_noalloc.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    lib.mb_sample_noalloc.restype = ctypes.c_int
    lib.mb_noalloc_strerror.argtypes = [ctypes.c_int]
    lib.mb_noalloc_strerror.restype = ctypes.c_char_p
    return lib


def pack(rows):
    from mashbox_b200.sampling.sampler import ROW
    packed = np.zeros(len(rows), ROW)
    for i, r in enumerate(rows):
        packed[i] = (r.get("temperature", 0.0), r.get("top_p", 1.0), r.get("min_p", 0.0), r.get("rep", 1.0),
                     r.get("freq", 0.0), r.get("pres", 0.0), r.get("top_k", 0), r.get("slot", -1), r.get("seed", 0), 0,
                     r.get("step", 0), i)
    return torch.from_numpy(packed.view(np.uint8).copy()).to(DEV)


def test_no_alloc_sampling_equals_the_ordinary_entry_point_twice_in_a_row():
    import mashbox_b200.ops as K
    lib = library()
    g = torch.Generator().manual_seed(21)
    stream = torch.cuda.current_stream().cuda_stream
    calls = [  # (vocab, rows): the second call is smaller and sharper, so stale scratch of the first would show
        (1009, [dict(temperature=0.9, top_k=50, seed=1), dict(), dict(temperature=1.2, top_p=0.7, seed=2, step=3),
                dict(temperature=0.8, min_p=0.1, rep=1.3, slot=1, seed=4)]),
        (257, [dict(temperature=0.5, top_k=3, top_p=0.9, seed=9, step=1), dict(temperature=1.0, seed=5)])]
    for call, (vocab, rows) in enumerate(calls):
        n = len(rows)
        logits = (3 * torch.randn(n, vocab, generator=g)).to(DEV)
        params = pack(rows)
        state = lambda: (torch.zeros(2, vocab, dtype=torch.int32, device=DEV),
                         torch.zeros(2, vocab, dtype=torch.uint8, device=DEV))
        cnt_a, seen_a = state()
        cnt_b, seen_b = state()
        seen_a[1, :40] = 1
        seen_b[1, :40] = 1
        want = torch.empty(n, dtype=torch.int32, device=DEV)
        K.sample(logits, torch.empty(n, vocab, device=DEV), params, cnt_a, seen_a, n, want)
        got = torch.full((n,), -1, dtype=torch.int32, device=DEV)
        torch.cuda.synchronize()
        before = torch.cuda.mem_get_info()[0]       # the driver's count: a cudaMalloc by anyone would show here
        rc = lib.mb_sample_noalloc(logits.data_ptr(), params.data_ptr(), cnt_b.data_ptr(), seen_b.data_ptr(), n, vocab,
                                   got.data_ptr(), stream)
        assert rc == 0, lib.mb_noalloc_strerror(rc)
        torch.cuda.synchronize()
        # The first call on a device is when the driver loads the library's image, the fixed 2 MiB array included;
        # from then on a call changes nothing.
        spent = before - torch.cuda.mem_get_info()[0]
        assert spent == 0 if call else 0 <= spent <= 8 << 20, spent
        assert got.tolist() == want.tolist()
        assert torch.equal(cnt_a, cnt_b) and torch.equal(seen_a, seen_b)


def test_no_alloc_sampling_refuses_what_does_not_fit():
    lib = library()
    x = torch.zeros(8, 16, device=DEV)
    out = torch.zeros(8, dtype=torch.int32, device=DEV)
    params = pack([dict()] * 8)
    args = (x.data_ptr(), params.data_ptr(), None, None)
    too_many = lib.mb_sample_noalloc(*args, lib.mb_noalloc_max_rows() + 1, 16, out.data_ptr(), None)
    too_wide = lib.mb_sample_noalloc(*args, 1, lib.mb_noalloc_max_vocab() + 1, out.data_ptr(), None)
    assert too_many == too_wide == -3 and b"beyond the fixed scratch" in lib.mb_noalloc_strerror(too_many)
    assert lib.mb_sample_noalloc(None, params.data_ptr(), None, None, 1, 16, out.data_ptr(), None) == -4
    assert b"null pointer" in lib.mb_noalloc_strerror(-4)
    cnt = torch.zeros(2, 16, dtype=torch.int32, device=DEV)
    assert lib.mb_sample_noalloc(x.data_ptr(), params.data_ptr(), cnt.data_ptr(), None, 1, 16, out.data_ptr(), None) == -4
