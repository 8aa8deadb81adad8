"""CPU: the selection-order routines compiled into the library (the same header the device kernels use)
return exactly the index lists of torch.topk on the host, ties included."""
import ctypes as C

import numpy as np
import pytest
import torch


def _lib():
    from coda_gqa_l_b200 import _lib
    return _lib.lib


def _topk(v: torch.Tensor, k: int, largest: bool, sorted_: bool):
    out = np.zeros(max(k, 1), dtype=np.int32)
    if v.dtype == torch.float32:
        a = np.ascontiguousarray(v.numpy(), dtype=np.float32)
        rc = _lib().coda_b200_host_topk_f32(a.ctypes.data, v.numel(), k, int(largest), int(sorted_), out.ctypes.data)
    else:
        a = np.ascontiguousarray(v.numpy(), dtype=np.int64)
        rc = _lib().coda_b200_host_topk_i64(a.ctypes.data, v.numel(), k, int(largest), int(sorted_), out.ctypes.data)
    assert rc == 0
    return out[:k].tolist()


def _gates(mode: int, n: int, g: torch.Generator) -> torch.Tensor:
    if mode == 0:
        return torch.full((n,), 0.11920292)                        # default constant gate
    if mode == 1:
        return torch.rand(n, generator=g)
    if mode == 2:
        return torch.randint(0, 3, (n,), generator=g).float()      # heavy ties
    v = torch.rand(n, generator=g)
    v[torch.rand(n, generator=g) < 0.5] = 0.5
    return v


@pytest.mark.parametrize("n", [1, 2, 3, 5, 8, 31, 64, 65, 127, 128, 192, 256, 257, 512, 1000, 1024, 4096])
def test_gate_selection_order(n):
    g = torch.Generator().manual_seed(n)
    for k in (1, 2, 7, 8, 9, 16, 17, 33, 63, 64, 65):
        if k > n:
            continue
        for mode in range(4):
            v = _gates(mode, n, g)
            for largest, sorted_ in ((True, False), (True, True), (False, False), (False, True)):
                ref = torch.topk(v.view(1, n), k, dim=1, largest=largest, sorted=sorted_)[1][0].tolist()
                assert _topk(v, k, largest, sorted_) == ref, (n, k, mode, largest, sorted_)


@pytest.mark.parametrize("Me", [4, 8, 16, 32, 64, 128, 256])
def test_lru_victim_order(Me):
    g = torch.Generator().manual_seed(Me)
    for k in (1, 2, 4, 8, 16, 18, 32):
        if k > Me:
            continue
        for mode in range(3):
            for _ in range(4):
                if mode == 0:
                    v = torch.full((Me,), -(2 ** 62), dtype=torch.int64)
                else:
                    v = torch.randint(0, 1000, (Me,), generator=g)
                    if mode == 2:
                        v[torch.rand(Me, generator=g) < 0.4] = -(2 ** 62)
                ref = torch.topk(v.view(1, Me), k, dim=1, largest=False, sorted=True)[1][0].tolist()
                assert _topk(v, k, False, True) == ref, (Me, k, mode)


def test_known_answers():
    """Index lists measured on the host top-k for the shapes the default configurations hit."""
    const = lambda n: torch.full((n,), 0.11920292)  # noqa: E731
    assert _topk(const(256), 64, True, False)[:9] == [160, 191, 190, 189, 188, 187, 186, 185, 184]
    assert _topk(const(256), 8, True, False) == [172, 169, 170, 171, 174, 175, 168, 173]
    assert _topk(const(128), 64, True, False)[:4] == [96, 65, 66, 67]
    unused = lambda n: torch.full((n,), -(2 ** 62), dtype=torch.int64)  # noqa: E731
    assert _topk(unused(64), 8, False, True) == [44, 41, 42, 43, 46, 47, 40, 45]
    assert _topk(unused(32), 8, False, True) == [20, 23, 22, 21, 18, 17, 24, 19]
