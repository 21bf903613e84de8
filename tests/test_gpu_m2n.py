"""Mesh-to-mesh resharding between GPUs (device buffers, grouped send / receive kernels)."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402
from test_m2n import DistTensor, Mesh, _slices  # noqa: E402

pytestmark = pytest.mark.gpu


def _rank(rank, nranks, uid, shape_global, src_mesh, dst_mesh, use_window=False):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator, _lib, mem_alloc
    from nccl_b200.core import FP32
    from nccl_b200.utils.perf import tensor_at
    comm = Communicator(nranks, rank, uid)
    lib = comm.lib
    win = None
    if use_window:
        # source tiles live in a registered window (with some bytes in front, so the tile offset is not zero)
        nbytes = int(np.prod(shape_global)) * 4 + 4096
        base = mem_alloc(nbytes)
        pool = tensor_at(base, nbytes)
        win = comm.register_window(pool)
    lib.ncclReshardWithWindow.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(DistTensor), ctypes.POINTER(DistTensor), ctypes.c_void_p]
    g = torch.arange(int(np.prod(shape_global)), dtype=torch.float32).reshape(shape_global)
    keep = []

    def side(mesh, fill):
        m = Mesh((ctypes.c_int * 2)(*mesh[0]), mesh[1], (ctypes.c_int * 2)(*mesh[2]))
        sl = _slices(mesh, shape_global, rank)
        tile_shape = list(shape_global)
        for a in range(2):
            if mesh[2][a] >= 0:
                tile_shape[mesh[2][a]] //= mesh[0][a]
        tile = None
        if sl is not None and fill and use_window:
            numel = int(np.prod(tile_shape))
            tile = pool[1024 * (1 + rank % 2):1024 * (1 + rank % 2) + numel * 4].view(torch.float32).view(tile_shape)
            tile.copy_(g[sl])
        elif sl is not None:
            tile = g[sl].contiguous().cuda() if fill else torch.full(tile_shape, -1.0, device="cuda")
        keep.append((m, tile))
        return DistTensor(tile.data_ptr() if tile is not None else None, (ctypes.c_size_t * 3)(*(tile_shape + [1] * (3 - len(tile_shape)))),
                          len(shape_global), FP32, ctypes.pointer(m)), tile

    st, _ = side(src_mesh, True)
    dt, d_tile = side(dst_mesh, False)
    torch.cuda.synchronize()
    for _ in range(2 if use_window else 1):   # the second call reuses the run list buffer and the barrier epochs
        _lib.check(lib.ncclReshardWithWindow(comm.handle, win, ctypes.byref(st), ctypes.byref(dt), torch.cuda.current_stream().cuda_stream),
                   "ncclReshardWithWindow", lib)
    torch.cuda.synchronize()
    out = None if d_tile is None else d_tile.cpu().numpy()
    assert comm.async_error() == 0
    comm.destroy()
    return out


@pytest.mark.parametrize("shape,src,dst", [((64, 96), ((2, 1), 0, (0, -1)), ((2, 1), 0, (1, -1))),      # rows -> columns on the same two GPUs
                                            ((32, 8, 16), ((1, 2), 0, (-1, 2)), ((2, 1), 0, (0, -1)))])  # 3-D, innermost -> outermost
@pytest.mark.parametrize("use_window", [False, True])
def test_reshard_two_gpus(shape, src, dst, use_window):
    """Without a window the runs move as grouped send / receive; with the source tiles in a registered window every
    destination rank pulls its runs with one kernel."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = run_ranks(_rank, 2, args=(shape, src, dst, use_window), timeout=200)
    g = np.arange(int(np.prod(shape)), dtype=np.float32).reshape(shape)
    for r in range(2):
        np.testing.assert_array_equal(res[r], g[_slices(dst, shape, r)])
