"""The allocation-free argmax entry point, called the way a host without torch's allocator would call it:
through its exported C symbol, with raw device pointers.

Such callers exist because some code may not allocate device memory at all: a host that fixes its
memory budget at start-up and forbids allocation afterwards, or a process that loads this library
from C without torch and so has no allocator to take scratch memory from. ``slb_argmax_static`` keeps its scratch memory in a fixed array inside the library, so the
caller passes logits and output only. Here its result is compared with the ordinary entry point's
(which takes scratch memory from the caller) on two calls in a row, the second with other data and
fewer rows, so that a result which leaned on what the first call left in the shared array would show.
This file is collected last on purpose: if it fails, every other test has already run.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_argmax_matches_the_ordinary_one_twice_in_a_row():
    from sleuth_b200.kernels import library
    dll = ctypes.CDLL(str(library.build(verbose=False)))            # the exported C symbols, nothing else
    P, L, I = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    dll.slb_argmax_static.argtypes = [P, L, I, I, P, P]
    dll.slb_argmax_static.restype = I
    dll.slb_argmax.argtypes = [P, L, I, I, P, P, L, P]
    dll.slb_argmax.restype = I
    dll.slb_last_error.restype = ctypes.c_char_p
    dll.slb_argmax_static_max_rows.restype = I

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(0)
    for rows, vocab, limit in ((37, 151936, 151936), (5, 1000, 777)):
        logits = torch.randn(rows, vocab, generator=g)
        logits[0, limit // 2] = logits[0, limit - 1] = 60.0             # a tie: the lower index must win
        logits = logits.to(dev)
        ours = torch.full((rows,), -1, dtype=torch.int32, device=dev)
        theirs = torch.full((rows,), -1, dtype=torch.int32, device=dev)
        scratch = torch.empty(2 * rows * 64, dtype=torch.int32, device=dev)
        rc = dll.slb_argmax_static(logits.data_ptr(), logits.stride(0), rows, limit, ours.data_ptr(), stream)
        assert rc == 0, dll.slb_last_error().decode()
        rc = dll.slb_argmax(logits.data_ptr(), logits.stride(0), rows, limit, theirs.data_ptr(), scratch.data_ptr(),
                            scratch.numel(), stream)
        assert rc == 0, dll.slb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.equal(ours, theirs)                                 # integer results: equal, not merely close
        assert ours.cpu().tolist() == logits[:, :limit].argmax(-1).cpu().tolist()
        assert int(ours[0]) == limit // 2

    too_many = dll.slb_argmax_static_max_rows() + 1
    rc = dll.slb_argmax_static(logits.data_ptr(), logits.stride(0), too_many, 10, ours.data_ptr(), stream)
    assert rc != 0 and str(too_many - 1) in dll.slb_last_error().decode()
