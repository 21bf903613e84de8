"""Programs written against the reference's Python bindings run over this library with their spelling
(``Communicator.init``, ``allreduce(send, recv, op, stream=)``, ``group()``, ...): two host-memory ranks."""
import numpy as np
import pytest

from mp_util import run_ranks

BASE = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo"}


def _rank(rank, nranks, uid):
    import nccl_b200.nccl4py.core as nccl
    comm = nccl.Communicator.init(nranks, rank, nccl.UniqueId(uid))
    assert comm.is_valid and comm.nranks == nranks and comm.rank == rank
    x = np.full(1000, rank + 1.0, dtype=np.float32)
    y = np.zeros_like(x)
    comm.allreduce(x, y, nccl.SUM)
    g = np.zeros(nranks * 10, dtype=np.float32)
    comm.allgather(x[:10], g)
    r = np.zeros(nranks * 4, dtype=np.float32)
    comm.reduce(np.arange(nranks * 4, dtype=np.float32), r, nccl.MAX, root=0)
    rs = np.zeros(5, dtype=np.float32)
    comm.reduce_scatter(np.ones(nranks * 5, dtype=np.float32) * (rank + 1), rs, nccl.SUM)
    b = np.full(7, float(rank), dtype=np.float32)
    comm.broadcast(b, b, root=nranks - 1)
    peer = (rank + 1) % nranks
    got = np.zeros(3, dtype=np.float32)
    with nccl.group():
        comm.send(np.full(3, 10.0 + rank, dtype=np.float32), peer)
        comm.recv(got, (rank - 1) % nranks)
    sub = comm.split(color=0, key=rank)
    s = np.ones(4, dtype=np.float32)
    sub.allreduce(s, s, nccl.SUM)
    sub.destroy()
    assert comm.get_async_error() == 0
    version = nccl.get_version()
    comm.destroy()
    return float(y[0]), float(g[-1]), float(r[-1]) if rank == 0 else None, float(rs[0]), float(b[0]), float(got[0]), float(s[0]), version


def test_reference_binding_spelling_on_host_ranks():
    n = 2
    res = run_ranks(_rank, n, env=BASE)
    tot = n * (n + 1) / 2
    for r in range(n):
        y, g, red, rs, b, got, s, version = res[r]
        assert y == tot and g == n and rs == tot and b == n - 1 and got == 10.0 + (r - 1) % n and s == n
        assert version >= 23000
        if r == 0:
            assert red == n * 4 - 1


REFERENCE_METHODS = """init init_all initialize split shrink get_unique_id grow destroy abort finalize revoke suspend resume ptr is_valid nranks
device rank cuda_dev nvml_dev device_api_support multimem_support gin_type n_lsa_teams host_rma_support railed_gin_type send recv wait_signal
signal put_signal allreduce broadcast reduce allgather reduce_scatter alltoall gather scatter register_buffer register_window
create_pre_mul_sum create_dev_comm close_all_resources get_last_error get_async_error get_mem_stat""".split()


def test_every_public_name_of_the_reference_communicator_exists():
    """The public methods and properties of the reference's ``nccl.core.Communicator`` (listed above; re-read from the
    reference tree when it is checked out next to this repository) all exist here under the same names."""
    import os
    import re
    import nccl_b200.nccl4py.core as nccl
    names = set(REFERENCE_METHODS)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(os.environ.get("NCCL_REFERENCE_DIR", os.path.join(os.path.dirname(root), "reference")), "bindings", "nccl4py", "nccl", "core",
                       "communicator.py")
    if os.path.exists(src):
        names |= {m for m in re.findall(r"^    def ([a-z][a-z0-9_]*)\(", open(src).read(), re.M)}
    missing = sorted(n for n in names if not hasattr(nccl.Communicator, n))
    assert not missing, missing


def _props_rank(rank, nranks, uid):
    import nccl_b200.nccl4py.core as nccl
    comm = nccl.Communicator.init(nranks, rank, nccl.UniqueId(uid))
    out = (comm.n_lsa_teams, comm.gin_type, comm.railed_gin_type, comm.host_rma_support, comm.device_api_support)
    comm.destroy()
    return out


def test_property_queries_on_host_ranks():
    res = run_ranks(_props_rank, 2, env=BASE)
    for r in range(2):
        n_lsa, gin, railed, rma, devapi = res[r]
        assert gin == 0 and railed == 0 and not devapi and n_lsa >= 1 and rma in (True, False)


EP_NAMES = """Algorithm AllocConfig AllocFn CombineConfig CombineInputs CombineOutputs DispatchConfig DispatchInputs DispatchOutputs FreeFn
get_lib_path get_lib_version Group GroupConfig Handle HandleConfig Layout LayoutInfo PassDir Tensor""".split()


def test_expert_parallel_module_has_the_reference_names():
    """Every name the reference's ``nccl.ep`` exports exists in ``nccl_b200.nccl4py.ep``, with the same record fields and the
    same methods on groups and handles (re-read from the reference tree when it is checked out next to this repository)."""
    import dataclasses
    import os
    import re
    import nccl_b200.nccl4py.ep as ep
    names = set(EP_NAMES)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.path.join(os.environ.get("NCCL_REFERENCE_DIR", os.path.join(os.path.dirname(root), "reference")), "bindings", "nccl4py", "nccl", "ep")
    methods = {"Group": {"create", "create_handle", "destroy", "ptr"}, "Handle": {"update", "dispatch", "combine", "complete", "destroy", "ptr"}}
    if os.path.isdir(ref):
        m = re.search(r"__all__ = \[(.*?)\]", open(os.path.join(ref, "__init__.py")).read(), re.S)
        names |= set(re.findall(r'"(\w+)"', m.group(1)))
        for cls, f in (("Group", "group.py"), ("Handle", "handle.py")):
            methods[cls] |= set(re.findall(r"^    def ([a-z][a-z0-9_]*)\(", open(os.path.join(ref, f)).read(), re.M))
    assert not sorted(n for n in names if not hasattr(ep, n))
    for cls, ms in methods.items():
        assert not sorted(m for m in ms if not hasattr(getattr(ep, cls), m)), cls
    assert [f.name for f in dataclasses.fields(ep.GroupConfig)] == ["algorithm", "num_experts", "max_dispatch_tokens_per_rank", "max_recv_tokens_per_rank",
        "max_token_bytes", "rdma_buffer_size", "num_qp_per_rank", "num_channels", "max_num_sms", "alloc", "enable_mask", "timeout_ns"]
    assert [f.name for f in dataclasses.fields(ep.DispatchOutputs)] == ["tokens", "topk_weights", "scales", "topk_idx"]
    assert [f.name for f in dataclasses.fields(ep.LayoutInfo)] == ["expert_counters", "src_rank_counters", "expert_offsets", "recv_total_counter"]
    assert (ep.Layout.EXPERT_MAJOR, ep.Layout.RANK_MAJOR, ep.Layout.FLAT) == (1, 2, 3) and ep.Algorithm.LOW_LATENCY == 0 and ep.PassDir.BWD == 1


def test_expert_parallel_tensor_descriptor_and_version():
    import numpy as np
    import nccl_b200.nccl4py.ep as ep
    a = np.zeros((6, 8), dtype=np.int64)
    t = ep.Tensor(a)
    assert t.ndim == 2 and t.sizes == (6, 8) and t.data == a.ctypes.data and t.ptr != 0 and t.buffer is a
    major, minor, patch = ep.get_lib_version()
    assert (major, minor, patch) >= (0, 1, 0)
    assert ep.get_lib_path().name == "libnccl_b200.so"
    li = ep.LayoutInfo(expert_counters=t)._struct()
    assert li.expert_counters.contents.data == a.ctypes.data and not li.expert_offsets


def test_expert_parallel_group_refuses_host_communicators():
    """Creating a group goes through ncclEpCreateGroup with the record's fields; on a host-memory communicator the library refuses."""
    res = run_ranks(_ep_group_rank, 2, env=BASE)
    assert res[0] == res[1] == "refused"


def _ep_group_rank(rank, nranks, uid):
    import nccl_b200.nccl4py.core as nccl
    import nccl_b200.nccl4py.ep as ep
    from nccl_b200._lib import NcclError
    comm = nccl.Communicator.init(nranks, rank, nccl.UniqueId(uid))
    try:
        ep.Group.create(comm, ep.GroupConfig(num_experts=8, max_dispatch_tokens_per_rank=16, max_token_bytes=256))
        out = "created"
    except NcclError:
        out = "refused"
    comm.destroy()
    return out


def test_version_report_names_the_loaded_library(capsys):
    import nccl_b200.nccl4py as nccl
    v = nccl.get_version()
    assert v.nccl is not None and v.nccl.version >= (2, 30, 0) and v.nccl.path.name == "libnccl_b200.so"
    assert v.nccl.cuda_variant is not None and v.nccl.cuda_variant[0] >= 12
    assert v.nccl_ep is not None and v.nccl_ep.version >= (0, 1, 0)
    nccl.show_versions()
    out = capsys.readouterr().out
    assert "libnccl" in out and "+cuda" in out and "libnccl_b200.so" in out


def test_interop_modules_describe_tensors_and_report_missing_frameworks():
    import pytest
    import torch
    from nccl_b200.nccl4py.core.interop import torch as nt
    from nccl_b200.nccl4py.core.interop import cupy as nc
    t = torch.zeros(3, 5, dtype=torch.bfloat16)
    ptr, n, dt, dev = nt.resolve_tensor(t)
    assert (ptr, n, dt, dev) == (t.data_ptr(), 15, 9, -1)
    with pytest.raises(ValueError):
        nt.resolve_tensor(torch.zeros(4, 4)[:, ::2])
    with pytest.raises(ValueError):
        nt.empty(4, morder="X")
    try:
        import cupy  # noqa: F401
    except ImportError:
        with pytest.raises(ModuleNotFoundError):
            nc.empty((4,))


@pytest.mark.gpu
def test_torch_tensor_in_library_memory_can_be_registered():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    import nccl_b200.nccl4py.core as nccl
    from nccl_b200.nccl4py.core.interop import torch as nt
    x = nt.empty(1024, 256, dtype=torch.float32)
    f = nt.empty(8, 4, dtype=torch.float16, morder="F")
    assert x.is_cuda and x.shape == (1024, 256) and x.is_contiguous() and f.stride() == (1, 8)
    x.fill_(3.0)
    comm = nccl.Communicator.init(1, 0, nccl.get_unique_id())
    win = comm.register_window(x)
    y = nt.empty(1024, 256, dtype=torch.float32)
    comm.allreduce(x, y, nccl.SUM)
    torch.cuda.synchronize()
    assert float(y.sum()) == 3.0 * 1024 * 256
    win.close()
    comm.destroy()
    del x, y, f
