"""Expert-parallel MoE dispatch / combine on torch tensors (wraps the ncclEp* C API).

    ep = ExpertParallel(comm, num_experts=256, max_tokens=4096, hidden=7168)
    toks, scales, counts = ep.dispatch(x, topk_idx, topk_weights, fp8=True)
        # toks [E_local, n*max_tokens, hidden] (e4m3 bytes), scales [E_local, n*max_tokens, hidden/128], counts [E_local]
    y = experts(toks, scales, counts)           # bf16 [E_local, n*max_tokens, hidden]
    out = ep.combine(y)                         # bf16 [tokens, hidden]: sum_k w[t,k] * y(expert k of t)

Layouts with one copy of a token per destination rank instead of one per expert (fewer bytes when a token selects
several experts of one rank): ``layout="rank_major"`` gives toks [n, max_tokens, hidden] (row = source rank, token
index) and ``layout="flat"`` gives the received tokens packed as [n*max_tokens, hidden]; both also return the routing
rows ``ep.recv_topk_idx`` (expert ids that are local to this rank, else -1) and ``ep.recv_topk_weights``. The caller
applies its local experts and the weights and gives one pre-reduced row per received token to ``combine``.
"""
import ctypes

from .. import _lib
from ..core import BF16, FP32, FP8_E4M3, INT32, INT64

EP_MAGIC = 0xC00FFFEE
TENSOR_MAGIC = 0xCAFECAFE


class EpTensor(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint), ("magic", ctypes.c_uint), ("ndim", ctypes.c_uint), ("datatype", ctypes.c_int),
                ("data", ctypes.c_void_p), ("win_hdl", ctypes.c_void_p), ("win_offset", ctypes.c_uint64),
                ("sizes", ctypes.POINTER(ctypes.c_size_t))]


class AllocCfg(ctypes.Structure):
    _fields_ = [("alloc_fn", ctypes.c_void_p), ("free_fn", ctypes.c_void_p), ("context", ctypes.c_void_p)]


class GroupCfg(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint), ("magic", ctypes.c_uint), ("version", ctypes.c_uint), ("algorithm", ctypes.c_int),
                ("num_experts", ctypes.c_uint), ("max_dispatch_tokens_per_rank", ctypes.c_uint), ("max_recv_tokens_per_rank", ctypes.c_uint),
                ("max_token_bytes", ctypes.c_uint), ("rdma_buffer_size", ctypes.c_ulong), ("num_qp_per_rank", ctypes.c_uint),
                ("num_channels", ctypes.c_uint), ("max_num_sms", ctypes.c_uint), ("alloc", AllocCfg), ("enable_mask", ctypes.c_uint),
                ("timeout_ns", ctypes.c_uint64)]


class LayoutInfo(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint), ("magic", ctypes.c_uint), ("expert_counters", ctypes.POINTER(EpTensor)),
                ("src_rank_counters", ctypes.POINTER(EpTensor)), ("expert_offsets", ctypes.POINTER(EpTensor)),
                ("recv_total_counter", ctypes.POINTER(EpTensor))]


class DispIn(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint), ("magic", ctypes.c_uint), ("tokens", ctypes.POINTER(EpTensor)),
                ("topk_weights", ctypes.POINTER(EpTensor)), ("scales", ctypes.POINTER(EpTensor))]


class DispOut(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint), ("magic", ctypes.c_uint), ("tokens", ctypes.POINTER(EpTensor)),
                ("topk_weights", ctypes.POINTER(EpTensor)), ("scales", ctypes.POINTER(EpTensor)), ("topk_idx", ctypes.POINTER(EpTensor))]


class DispCfg(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint), ("magic", ctypes.c_uint), ("send_only", ctypes.c_uint), ("round_scales", ctypes.c_uint), ("pass_direction", ctypes.c_int)]


class CombCfg(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint), ("magic", ctypes.c_uint), ("send_only", ctypes.c_uint), ("pass_direction", ctypes.c_int)]


class CombIO(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint), ("magic", ctypes.c_uint), ("tokens", ctypes.POINTER(EpTensor)), ("topk_weights", ctypes.POINTER(EpTensor))]


def _tensor(t, code):
    sizes = (ctypes.c_size_t * t.dim())(*t.shape)
    et = EpTensor(ctypes.sizeof(EpTensor), TENSOR_MAGIC, t.dim(), code, t.data_ptr(), None, 0, sizes)
    et._keep = (sizes, t)
    return et


def _hdr(s):
    s.size = ctypes.sizeof(s)
    s.magic = EP_MAGIC
    return s


class ExpertParallel:
    LAYOUTS = {"expert_major": 1, "rank_major": 2, "flat": 3}

    def __init__(self, comm, num_experts, max_tokens, hidden, max_sms=0, timeout_ms=0, enable_mask=False, layout="expert_major"):
        import torch
        self.torch = torch
        self.layout = layout
        self.layout_code = self.LAYOUTS[layout]
        self.comm, self.lib = comm, comm.lib
        self.E, self.n, self.H, self.max_tokens = num_experts, comm.nranks, hidden, max_tokens
        self.El = num_experts // comm.nranks
        self.cap = comm.nranks * max_tokens
        L = self.lib
        vp, pvp = ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)
        L.ncclEpCreateGroup.argtypes = [pvp, vp, ctypes.POINTER(GroupCfg)]
        L.ncclEpGroupDestroy.argtypes = [vp]
        L.ncclEpCreateHandle.argtypes = [pvp, vp, ctypes.c_int, ctypes.POINTER(EpTensor), vp, vp, vp]
        L.ncclEpUpdateHandle.argtypes = [vp, ctypes.POINTER(EpTensor), vp, vp]
        L.ncclEpHandleDestroy.argtypes = [vp]
        L.ncclEpDispatch.argtypes = [vp, ctypes.POINTER(DispIn), ctypes.POINTER(DispOut), ctypes.POINTER(LayoutInfo), ctypes.POINTER(DispCfg), vp]
        L.ncclEpCombine.argtypes = [vp, ctypes.POINTER(CombIO), ctypes.POINTER(CombIO), ctypes.POINTER(CombCfg), vp]
        L.ncclEpComplete.argtypes = [vp, vp, vp]
        L.ncclEpMaskQuery.argtypes = [vp, ctypes.POINTER(ctypes.c_int), vp]
        L.ncclEpMaskUpdate.argtypes = [vp, ctypes.POINTER(ctypes.c_int), vp]
        L.ncclEpMaskClean.argtypes = [vp, vp]
        cfg = _hdr(GroupCfg())
        cfg.version = 1
        cfg.num_experts = num_experts
        cfg.max_dispatch_tokens_per_rank = max_tokens
        cfg.max_token_bytes = hidden * 2
        cfg.max_num_sms = max_sms
        cfg.timeout_ns = timeout_ms * 1000000
        cfg.enable_mask = 1 if enable_mask else 0
        g = ctypes.c_void_p()
        _lib.check(L.ncclEpCreateGroup(ctypes.byref(g), comm.handle, ctypes.byref(cfg)), "ncclEpCreateGroup", L)
        self.group = g
        self.handle = None
        self._keep = None

    def destroy(self):
        if self.handle:
            self.lib.ncclEpHandleDestroy(self.handle)
            self.handle = None
        if self.group:
            self.lib.ncclEpGroupDestroy(self.group)
            self.group = None

    def _stream(self):
        return self.torch.cuda.current_stream().cuda_stream

    def complete(self):
        """Runs the receiving half of the last ``send_only`` dispatch / combine."""
        _lib.check(self.lib.ncclEpComplete(self.handle, None, self._stream()), "ncclEpComplete", self.lib)

    def mask(self):
        """Which ranks this rank leaves out (1 = left out)."""
        m = (ctypes.c_int * self.n)()
        _lib.check(self.lib.ncclEpMaskQuery(self.group, m, self._stream()), "ncclEpMaskQuery", self.lib)
        return list(m)

    def set_mask(self, mask):
        m = (ctypes.c_int * self.n)(*mask)
        _lib.check(self.lib.ncclEpMaskUpdate(self.group, m, self._stream()), "ncclEpMaskUpdate", self.lib)

    def clear_mask(self):
        _lib.check(self.lib.ncclEpMaskClean(self.group, self._stream()), "ncclEpMaskClean", self.lib)

    def dispatch(self, x, topk_idx, topk_weights, fp8=True, toks=None, scales=None, counts=None, send_only=False):
        """``send_only``: only queue the sends; ``complete()`` then waits for the peers' tokens and packs them
        (work queued in between overlaps the transfer)."""
        torch, L = self.torch, self.lib
        idx_t = _tensor(topk_idx, INT64)
        if self.handle is None:
            h = ctypes.c_void_p()
            _lib.check(L.ncclEpCreateHandle(ctypes.byref(h), self.group, self.layout_code, ctypes.byref(idx_t), None, None, self._stream()), "ncclEpCreateHandle", L)
            self.handle = h
        else:
            _lib.check(L.ncclEpUpdateHandle(self.handle, ctypes.byref(idx_t), None, self._stream()), "ncclEpUpdateHandle", L)
        lead = {"expert_major": (self.El, self.cap), "rank_major": (self.n, self.max_tokens), "flat": (self.cap,)}[self.layout]
        if toks is None:
            toks = torch.empty(*lead, self.H, dtype=torch.uint8 if fp8 else torch.bfloat16, device=x.device)
        if scales is None and fp8:
            scales = torch.empty(*lead, self.H // 128, dtype=torch.float32, device=x.device)
        if counts is None:
            counts = torch.zeros(self.El, dtype=torch.int32, device=x.device)
        xin, win = _tensor(x, BF16), _tensor(topk_weights, FP32)
        tout, cnt_t = _tensor(toks, FP8_E4M3 if fp8 else BF16), _tensor(counts, INT32)
        sout = _tensor(scales, FP32) if fp8 else None
        din = _hdr(DispIn())
        din.tokens, din.topk_weights = ctypes.pointer(xin), ctypes.pointer(win)
        dout = _hdr(DispOut())
        dout.tokens = ctypes.pointer(tout)
        if fp8:
            dout.scales = ctypes.pointer(sout)
        li = _hdr(LayoutInfo())
        li.expert_counters = ctypes.pointer(cnt_t)
        extra = None
        if self.layout != "expert_major":
            K = topk_idx.shape[1]
            self.recv_topk_idx = torch.empty(*lead, K, dtype=torch.int64, device=x.device)
            self.recv_topk_weights = torch.empty(*lead, K, dtype=torch.float32, device=x.device)
            self.recv_total = torch.zeros(1, dtype=torch.int32, device=x.device)
            extra = (_tensor(self.recv_topk_idx, INT64), _tensor(self.recv_topk_weights, FP32), _tensor(self.recv_total, INT32))
            dout.topk_idx, dout.topk_weights = ctypes.pointer(extra[0]), ctypes.pointer(extra[1])
            if self.layout == "flat":
                li.recv_total_counter = ctypes.pointer(extra[2])
        dcfg = _hdr(DispCfg())
        dcfg.send_only = 1 if send_only else 0
        _lib.check(L.ncclEpDispatch(self.handle, ctypes.byref(din), ctypes.byref(dout), ctypes.byref(li), ctypes.byref(dcfg), self._stream()), "ncclEpDispatch", L)
        self._keep = (topk_idx, topk_weights, idx_t, xin, win, tout, cnt_t, sout, extra)
        self.T = x.shape[0]
        return toks, scales, counts

    def combine(self, y, out=None, send_only=False):
        torch, L = self.torch, self.lib
        out = out if out is not None else torch.empty(self.T, self.H, dtype=torch.bfloat16, device=y.device)
        yin, oout = _tensor(y, BF16), _tensor(out, BF16)
        cin, cout = _hdr(CombIO()), _hdr(CombIO())
        cin.tokens, cout.tokens = ctypes.pointer(yin), ctypes.pointer(oout)
        ccfg = _hdr(CombCfg())
        ccfg.send_only = 1 if send_only else 0
        _lib.check(L.ncclEpCombine(self.handle, ctypes.byref(cin), ctypes.byref(cout), ctypes.byref(ccfg), self._stream()), "ncclEpCombine", L)
        self._keep_c = (yin, oout, y, out)
        return out
