"""The allocation-free indexer entry point against the regular one.

`kch_indexer_topk_static` exists for callers that may not allocate device memory while serving (a decode
loop inside a runtime with a frozen memory pool; a thread that must not enter the CUDA allocator): it keeps
its logits in an array built into the library instead of a caller-provided workspace.  It must pick exactly
the same blocks as `kch_indexer_topk`, also on a second call that finds the first call's logits still in the
array.  This file is collected last so that a run stopping at the first failure has already run every
other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, B, T, n, HI, DI):
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(B, T, HI, DI, generator=g), dim=-1).to(DEV).contiguous()
    k = torch.nn.functional.normalize(torch.randn(B, n, DI, generator=g), dim=-1).to(DEV).contiguous()
    w = (torch.randn(B, T, HI, generator=g) * 0.1).to(DEV).contiguous()
    return q, k, w


def _both(lib, q, k, w, topk, m, n_visible):
    from kch_b200 import _lib
    B, T, HI, DI = q.shape
    n = k.shape[1]
    stream = _lib.stream()
    ref = torch.empty(B, T, topk, dtype=torch.int32, device=DEV)
    nbytes = int(lib.kch_indexer_workspace_bytes(B, T, n, HI, DI))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    _lib.check(lib.kch_indexer_topk(_lib.ptr(q), _lib.ptr(k), _lib.ptr(w), _lib.ptr(ref), B, T, n, HI, DI, topk, 1.0,
                                    m, 0, n_visible, 0, 0, _lib.ptr(ws), nbytes, stream))
    out = torch.full((B, T, topk), -7, dtype=torch.int32, device=DEV)
    before = torch.cuda.memory_allocated()
    _lib.check(lib.kch_indexer_topk_static(_lib.ptr(q), _lib.ptr(k), _lib.ptr(w), _lib.ptr(out), B, T, n, HI, DI, topk,
                                           1.0, m, 0, n_visible, 0, stream))
    assert torch.cuda.memory_allocated() == before
    torch.cuda.synchronize()
    return ref.cpu(), out.cpu()


def test_static_indexer_matches_workspace_indexer_twice():
    from kch_b200 import _lib
    lib = _lib.load()
    assert lib.kch_indexer_topk_static_capacity() == 4 * 1024 * 1024
    # call 1: a prefill-shaped request (causal rule), call 2: a smaller decode-shaped request that finds
    # the logits of call 1 still in the built-in array
    q, k, w = _case(101, 2, 256, 192, 4, 64)
    ref, out = _both(lib, q, k, w, topk=48, m=4, n_visible=-1)
    assert torch.equal(ref, out)
    q, k, w = _case(102, 3, 1, 150, 4, 64)
    ref, out = _both(lib, q, k, w, topk=32, m=0, n_visible=97)
    assert torch.equal(ref, out)
    assert int((out >= 97).sum()) == 0 and int((out >= 0).sum()) == 3 * 32
    # call 3 repeats call 1's shape with new data: stale logits of call 2 must not leak in
    q, k, w = _case(103, 2, 256, 192, 4, 64)
    ref, out = _both(lib, q, k, w, topk=48, m=4, n_visible=-1)
    assert torch.equal(ref, out)


def test_static_indexer_other_kernel_paths():
    """The same comparison on the two other kernel combinations behind the entry point: an indexer width the
    tensor-core logits kernel does not serve (c_I = 32), and rows longer than 8192 blocks, whose select stages
    the row in shared memory instead of registers."""
    from kch_b200 import _lib
    lib = _lib.load()
    q, k, w = _case(104, 2, 96, 160, 3, 32)
    ref, out = _both(lib, q, k, w, topk=24, m=4, n_visible=-1)
    assert torch.equal(ref, out)
    q, k, w = _case(105, 1, 128, 8200, 4, 64)                    # 128 * 8200 logits < 4 Mi
    ref, out = _both(lib, q, k, w, topk=64, m=0, n_visible=8199)
    assert torch.equal(ref, out)
    assert int((out >= 8199).sum()) == 0 and int((out >= 0).sum()) == 128 * 64


def test_static_indexer_rejects_oversized_requests():
    from kch_b200 import _lib
    lib = _lib.load()
    cap = int(lib.kch_indexer_topk_static_capacity())
    dummy = torch.zeros(8, dtype=torch.float32, device=DEV)
    idx = torch.zeros(8, dtype=torch.int32, device=DEV)
    B, T, n = 1, 2049, 2048                                      # 2049 * 2048 logits > 4 Mi
    assert B * T * n > cap
    rc = lib.kch_indexer_topk_static(_lib.ptr(dummy), _lib.ptr(dummy), None, _lib.ptr(idx), B, T, n, 1, 8, 4, 1.0, 4, 0,
                                     -1, 0, _lib.stream())
    assert rc < 0
    with pytest.raises(ValueError, match="built-in scratch"):
        _lib.check(rc)
