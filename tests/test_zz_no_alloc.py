"""The allocation-free gradient-norm entry point (rte_grad_norm_multi_tensor_static).

Some embedders of this library cannot give it scratch memory and must not allocate any: they hold only the
parameter/gradient pointers a training framework handed them, and the framework's caching allocator owns the
rest of the GPU.  For them the library carries its own fixed scratch array.  This test drives that entry point
through the C ABI and checks it against the ordinary one (caller-supplied scratch) on two consecutive calls,
the second with different gradients, so stale contents of the shared array would show.
Collected last on purpose: a failure here cannot hide the results of the other GPU tests under `-x`.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _plan(shapes, gen, dev=DEV):
    from speedup_thingy_b200.ops import AdamWPlan

    entries = []
    for i, s in enumerate(shapes):
        p = torch.randn(s, generator=gen).to(dev)
        entries.append(dict(p=p, g=torch.zeros_like(p), m=torch.zeros_like(p), v=torch.zeros_like(p), shadow=None, lr_group=0))
    return AdamWPlan(entries, 1, dev), entries


@pytest.mark.parametrize("dev", ["cuda:0", "cuda:1"])
def test_static_scratch_grad_norm_matches_the_regular_entry_point_twice_in_a_row(dev):
    """`cuda:1` (skipped on a single-GPU machine): the array's device address is looked up per device, with that device
    current -- each GPU that loads the library carries its own copy of the array."""
    from speedup_thingy_b200.ops import CudaOps

    if int(dev.split(":")[1]) >= torch.cuda.device_count():
        pytest.skip("needs a second GPU")
    ops = CudaOps(dev)
    gen = torch.Generator().manual_seed(1234)
    plan, entries = _plan([(70_001,), (513, 129), (4096,), (3,)], gen, dev)
    partial = torch.zeros(plan.total_chunks, device=dev)
    for call, scale in enumerate((1.0, 0.01)):
        for e in entries:
            e["g"].copy_((torch.randn(e["g"].shape, generator=gen) * scale).to(dev))
        ref_sumsq, ref_clip = torch.zeros(1, device=dev), torch.zeros(1, device=dev)
        got_sumsq, got_clip = torch.full((1,), -1.0, device=dev), torch.full((1,), -1.0, device=dev)
        with torch.cuda.device(dev):
            ops.grad_norm(plan, partial, ref_sumsq, 1.0, ref_clip)
            ops.grad_norm_static(plan, got_sumsq, 1.0, got_clip)
        torch.cuda.synchronize(dev)
        host = sum(float(e["g"].double().pow(2).sum()) for e in entries)
        assert abs(float(ref_sumsq) - host) <= 1e-4 * host, call
        assert abs(float(got_sumsq) - float(ref_sumsq)) <= 1e-6 * float(ref_sumsq), call
        assert abs(float(got_clip) - float(ref_clip)) <= 1e-6, call


def test_static_scratch_rejects_tables_beyond_its_capacity():
    from speedup_thingy_b200 import _abi
    from speedup_thingy_b200.ops import CudaOps

    ops = CudaOps(DEV)
    plan, _ = _plan([(128,)], torch.Generator().manual_seed(0))
    out = torch.zeros(2, device=DEV)
    code = ops.lib.rte_grad_norm_multi_tensor_static(C.c_void_p(plan.table.data_ptr()), 65537,
                                                     C.c_void_p(plan.chunk_tensor.data_ptr()),
                                                     C.c_void_p(plan.chunk_index.data_ptr()), C.c_void_p(out.data_ptr()),
                                                     1.0, C.c_void_p(out[1:].data_ptr()), ops.stream)
    assert code == -7
    assert b"built-in scratch" in ops.lib.rte_status_string(code)
    torch.cuda.synchronize()
