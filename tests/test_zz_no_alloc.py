"""b200moe_permute_static: the permutation for callers that cannot pass scratch memory (a server whose device
memory pool is fixed at start-up, a plugin that only gets input and output buffers).  Called through the C ABI,
twice in a row, and compared bit for bit with b200moe_permute on the same inputs.  Collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_permute_static_matches_permute_twice():
    import torch_tpu_b200
    L = torch_tpu_b200.lib
    ops = torch_tpu_b200.ops
    lib = L.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.b200moe_permute_static_max_scratch_ints() == 65536
    for call, (T, k, E, seed) in enumerate([(8192, 8, 128, 1), (5000, 6, 256, 2), (300, 2, 8, 3)]):
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32).to(DEV)
        want_order, want_offs = ops.permute(ids, E)
        order = torch.full((T * k,), -7, dtype=torch.int32, device=DEV)
        offs = torch.full((E + 1,), -7, dtype=torch.int32, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        rc = lib.b200moe_permute_static(_ptr(order), _ptr(offs), _ptr(ids), T, k, E, _ptr(status), stream)
        assert rc == 0, L.error_string(rc)
        torch.cuda.synchronize()
        assert torch.equal(order, want_order), f"call {call}: sorted pairs differ"
        assert torch.equal(offs, want_offs), f"call {call}: offsets differ"
        assert int(status.item()) == 0


def test_permute_static_rejects_sizes_beyond_its_array():
    import torch_tpu_b200
    L = torch_tpu_b200.lib
    lib = L.lib()
    one = ctypes.c_void_p(256)
    # 1,000,000 pairs x 1024 experts needs ~1e6 ints of scratch: beyond the fixed 65536
    rc = lib.b200moe_permute_static(one, one, one, 125000, 8, 1024, None, None)
    assert rc == L.ESHAPE
    assert "unsupported size" in L.error_string(rc)
