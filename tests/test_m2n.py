"""Mesh-to-mesh resharding on CPU ranks: every destination tile must equal its slice of the global tensor."""
import ctypes

import numpy as np
import pytest

from mp_util import run_ranks

ENV = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo"}


class Mesh(ctypes.Structure):
    _fields_ = [("dims", ctypes.c_int * 2), ("startRank", ctypes.c_int), ("placement", ctypes.c_int * 2)]


class DistTensor(ctypes.Structure):
    _fields_ = [("dataPtr", ctypes.c_void_p), ("localShape", ctypes.c_size_t * 3), ("ndims", ctypes.c_int), ("dtype", ctypes.c_int),
                ("mesh", ctypes.POINTER(Mesh))]


def _slices(mesh, shape_global, rank):
    """numpy index of the tile of `rank` on a mesh description (dims, start, placement), or None."""
    dims, start, placement = mesh
    idx = rank - start
    if idx < 0 or idx >= dims[0] * dims[1]:
        return None
    coord = (idx // dims[1], idx % dims[1])
    sl = [slice(None)] * len(shape_global)
    for a in range(2):
        if placement[a] >= 0:
            td = placement[a]
            step = shape_global[td] // dims[a]
            sl[td] = slice(coord[a] * step, (coord[a] + 1) * step)
    return tuple(sl)


def _rank(rank, nranks, uid, shape_global, src_mesh, dst_mesh):
    from nccl_b200 import Communicator, _lib
    from nccl_b200.core import FP32
    comm = Communicator(nranks, rank, uid)
    lib = comm.lib
    lib.ncclReshardWithWindow.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(DistTensor), ctypes.POINTER(DistTensor), ctypes.c_void_p]
    g = np.arange(int(np.prod(shape_global)), dtype=np.float32).reshape(shape_global)

    def side(mesh, fill):
        m = Mesh((ctypes.c_int * 2)(*mesh[0]), mesh[1], (ctypes.c_int * 2)(*mesh[2]))
        sl = _slices(mesh, shape_global, rank)
        tile_shape = list(shape_global)
        for a in range(2):
            if mesh[2][a] >= 0:
                tile_shape[mesh[2][a]] //= mesh[0][a]
        tile = None
        if sl is not None:
            tile = np.ascontiguousarray(g[sl]) if fill else np.full(tile_shape, -1.0, dtype=np.float32)
        t = DistTensor(tile.ctypes.data if tile is not None else None, (ctypes.c_size_t * 3)(*(tile_shape + [1] * (3 - len(tile_shape)))),
                       len(shape_global), FP32, ctypes.pointer(m))
        return t, tile, m

    st, s_tile, sm = side(src_mesh, True)
    dt, d_tile, dm = side(dst_mesh, False)
    _lib.check(lib.ncclReshardWithWindow(comm.handle, None, ctypes.byref(st), ctypes.byref(dt), None), "ncclReshardWithWindow", lib)
    comm.destroy()
    return None if d_tile is None else d_tile


CASES = [
    # global shape, source mesh (dims, start, placement), destination mesh
    ((8, 6), ((2, 2), 0, (0, -1)), ((1, 2), 4, (-1, 1)), 6),        # 2 shards x 2 replicas over rows -> 2 column shards on other ranks
    ((8, 12), ((4, 1), 0, (0, -1)), ((2, 1), 0, (1, -1)), 4),       # same ranks on both sides: row shards -> column shards
    ((4, 6, 8), ((1, 2), 0, (-1, 2)), ((3, 1), 2, (1, -1)), 5),     # 3-D: innermost dimension sharded -> middle dimension sharded
    ((16,), ((2, 1), 0, (0, -1)), ((2, 2), 2, (-1, -1)), 6),        # 1-D shards -> fully replicated on four ranks
]


@pytest.mark.parametrize("shape,src,dst,n", CASES)
def test_reshard(shape, src, dst, n):
    res = run_ranks(_rank, n, args=(shape, src, dst), env=ENV, timeout=120)
    g = np.arange(int(np.prod(shape)), dtype=np.float32).reshape(shape)
    seen = 0
    for r in range(n):
        sl = _slices(dst, shape, r)
        if sl is None:
            assert res[r] is None
            continue
        np.testing.assert_array_equal(res[r], g[sl])
        seen += 1
    assert seen == dst[0][0] * dst[0][1]
