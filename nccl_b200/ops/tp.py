"""Fused tensor-parallel linear layers (bf16, tcgen05 GEMM fused with its collective).

    tp = TensorParallel(comm, max_rows=8192, max_cols=8192)
    y  = tp.gemm(x, w)                      # x [M,K], w [N,K] -> [M,N]
    y  = tp.gemm_reduce_scatter(x, w)       # row-parallel layer: [M,Ks] x [N,Ks] -> [M/n, N], summed over ranks
    xg = tp.alloc_gathered(M, K)            # symmetric activation buffer; fill rows of this rank
    y  = tp.all_gather_gemm(xg, w)          # column-parallel layer: gathers the rows while multiplying
"""
import ctypes

from .. import _lib


def _torch():
    import torch
    return torch


class TensorParallel:
    def __init__(self, comm, max_rows, max_cols):
        self.comm = comm
        self.lib = comm.lib
        L = self.lib
        L.ncclTpCreate.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)]
        L.ncclTpDestroy.argtypes = [ctypes.c_void_p]
        L.ncclTpAllocGathered.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)]
        L.ncclTpFreeGathered.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        sig = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        for name in ("ncclTpGemm", "ncclTpGemmReduceScatter", "ncclTpAllGatherGemm"):
            getattr(L, name).argtypes = sig
        h = ctypes.c_void_p()
        _lib.check(L.ncclTpCreate(comm.handle, max_rows, max_cols, ctypes.byref(h)), "ncclTpCreate", L)
        self.handle = h
        self._gathered = {}

    def destroy(self):
        if self.handle:
            self._gathered.clear()
            _lib.check(self.lib.ncclTpDestroy(self.handle), "ncclTpDestroy", self.lib)
            self.handle = None

    def _stream(self, stream):
        torch = _torch()
        return (stream or torch.cuda.current_stream()).cuda_stream

    @staticmethod
    def _check(x, w):
        torch = _torch()
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not x.is_contiguous() or not w.is_contiguous():
            raise ValueError("operands must be contiguous bf16 tensors")
        if x.shape[1] != w.shape[1]:
            raise ValueError("x [M,K] and w [N,K] must share K")

    def gemm(self, x, w, out=None, stream=None):
        torch = _torch()
        self._check(x, w)
        M, K = x.shape
        N = w.shape[0]
        out = out if out is not None else torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        _lib.check(self.lib.ncclTpGemm(self.handle, x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, self._stream(stream)), "ncclTpGemm", self.lib)
        return out

    def gemm_reduce_scatter(self, x, w, out=None, stream=None):
        torch = _torch()
        self._check(x, w)
        M, K = x.shape
        N = w.shape[0]
        n = self.comm.nranks
        out = out if out is not None else torch.empty(M // n, N, dtype=torch.bfloat16, device=x.device)
        rc = self.lib.ncclTpGemmReduceScatter(self.handle, x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, self._stream(stream))
        _lib.check(rc, "ncclTpGemmReduceScatter", self.lib)
        return out

    def alloc_gathered(self, rows, cols):
        """Collective. A [rows, cols] bf16 tensor in a symmetric window; each rank owns rows/n of it."""
        torch = _torch()
        from ..utils.perf import tensor_at
        p = ctypes.c_void_p()
        _lib.check(self.lib.ncclTpAllocGathered(self.handle, rows, cols, ctypes.byref(p)), "ncclTpAllocGathered", self.lib)
        t = tensor_at(p.value, rows * cols * 2).view(torch.bfloat16).view(rows, cols)
        self._gathered[t.data_ptr()] = p
        return t

    def all_gather_gemm(self, gathered, w, out=None, stream=None):
        torch = _torch()
        self._check(gathered, w)
        M, K = gathered.shape
        N = w.shape[0]
        out = out if out is not None else torch.empty(M, N, dtype=torch.bfloat16, device=w.device)
        rc = self.lib.ncclTpAllGatherGemm(self.handle, gathered.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, self._stream(stream))
        _lib.check(rc, "ncclTpAllGatherGemm", self.lib)
        return out

    # ------------------------------------------------------------------ block-scaled fp8 (e4m3)
    def _fp8_protos(self):
        if getattr(self, "_fp8_ready", False):
            return
        L, P, I = self.lib, ctypes.c_void_p, ctypes.c_int
        L.ncclTpQuantizeFp8.argtypes = [P, P, P, P, I, I, I, P]
        L.ncclTpGemmFp8.argtypes = [P, P, P, P, P, P, I, I, I, P]
        L.ncclTpGemmReduceScatterFp8.argtypes = [P, P, P, P, P, P, I, I, I, P]
        L.ncclTpAllocGatheredFp8.argtypes = [P, ctypes.c_size_t, ctypes.c_size_t, ctypes.POINTER(P), ctypes.POINTER(P)]
        L.ncclTpAllGatherGemmFp8.argtypes = [P, P, P, P, P, I, I, I, P]
        self._fp8_ready = True

    def quantize_fp8(self, x, block_rows=1, q=None, scales=None, stream=None):
        """bf16 [R, K] -> (e4m3 [R, K], fp32 scales). block_rows 1: activations, scales [K/128, R];
        block_rows 128: weights, scales [K/128, R/128]. x ~= q * scale."""
        torch = _torch()
        self._fp8_protos()
        R, K = x.shape
        if x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError("x must be a contiguous bf16 matrix")
        q = q if q is not None else torch.empty(R, K, dtype=torch.float8_e4m3fn, device=x.device)
        scales = scales if scales is not None else torch.empty(K // 128, R // block_rows, dtype=torch.float32, device=x.device)
        rc = self.lib.ncclTpQuantizeFp8(self.handle, x.data_ptr(), q.data_ptr(), scales.data_ptr(), R, K, block_rows, self._stream(stream))
        _lib.check(rc, "ncclTpQuantizeFp8", self.lib)
        return q, scales

    def gemm_fp8(self, xq, xs, wq, ws, out=None, stream=None):
        torch = _torch()
        self._fp8_protos()
        M, K = xq.shape
        N = wq.shape[0]
        out = out if out is not None else torch.empty(M, N, dtype=torch.bfloat16, device=xq.device)
        rc = self.lib.ncclTpGemmFp8(self.handle, xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), out.data_ptr(), M, N, K, self._stream(stream))
        _lib.check(rc, "ncclTpGemmFp8", self.lib)
        return out

    def gemm_reduce_scatter_fp8(self, xq, xs, wq, ws, out=None, stream=None):
        torch = _torch()
        self._fp8_protos()
        M, K = xq.shape
        N = wq.shape[0]
        out = out if out is not None else torch.empty(M // self.comm.nranks, N, dtype=torch.bfloat16, device=xq.device)
        rc = self.lib.ncclTpGemmReduceScatterFp8(self.handle, xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), out.data_ptr(), M, N, K,
                                                 self._stream(stream))
        _lib.check(rc, "ncclTpGemmReduceScatterFp8", self.lib)
        return out

    def alloc_gathered_fp8(self, rows, cols):
        """Collective. (e4m3 [rows, cols], fp32 scales [cols/128, rows]) in one symmetric window."""
        torch = _torch()
        self._fp8_protos()
        from ..utils.perf import tensor_at
        q, s = ctypes.c_void_p(), ctypes.c_void_p()
        _lib.check(self.lib.ncclTpAllocGatheredFp8(self.handle, rows, cols, ctypes.byref(q), ctypes.byref(s)), "ncclTpAllocGatheredFp8", self.lib)
        tq = tensor_at(q.value, rows * cols).view(torch.float8_e4m3fn).view(rows, cols)
        ts = tensor_at(s.value, cols // 128 * rows * 4).view(torch.float32).view(cols // 128, rows)
        self._gathered[tq.data_ptr()] = q
        return tq, ts

    def all_gather_gemm_fp8(self, gathered_q, wq, ws, out=None, stream=None):
        torch = _torch()
        self._fp8_protos()
        M, K = gathered_q.shape
        N = wq.shape[0]
        out = out if out is not None else torch.empty(M, N, dtype=torch.bfloat16, device=wq.device)
        rc = self.lib.ncclTpAllGatherGemmFp8(self.handle, gathered_q.data_ptr(), wq.data_ptr(), ws.data_ptr(), out.data_ptr(), M, N, K, self._stream(stream))
        _lib.check(rc, "ncclTpAllGatherGemmFp8", self.lib)
        return out
