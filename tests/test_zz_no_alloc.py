"""The allocation-free GEMV entry point against the regular one and the CPU oracle (runs last: file name sorts after the others).

Hosts that have given all of HBM to their own pools cannot let the library call cudaMalloc on the
decode path; ``prism_cuda_gemv_static_dev`` keeps its split-K scratch in a fixed array inside the
library.  Its result must equal ``prism_cuda_gemv_dev`` and the oracle's ``lut_gemv`` on the same inputs, call
after call, since every call reuses (and must re-initialise) the same scratch; and the device's free
memory must not move across a call.
"""
import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu


def test_static_scratch_gemv_matches_regular_entry_point():
    import torch

    import prism_engine_b200 as p
    from oracle import oracle as orc
    from prism_engine_b200 import synth

    be = p.CudaBackend(device=0)
    try:
        # split-K shapes (few row blocks, long K), and one whose K is not split at all (no scratch used)
        for (m, k) in [(896, 4864), (4864, 896), (128, 8192), (64 * 500, 256)]:
            pay = synth.make_payload(m, k, 4, seed=m + 3 * k)
            h = be.upload(f"static.{m}x{k}", pay, m, k)
            want = None
            for call in range(2):                                   # two calls in a row share the scratch
                x = synth.make_activation(k, seed=100 + call)
                xd = torch.from_numpy(x.view(np.int16)).cuda()
                y_ref = torch.zeros(m, dtype=torch.int16, device="cuda")
                y_new = torch.full((m,), 0x7E00, dtype=torch.int16, device="cuda")   # poison
                torch.cuda.synchronize()
                be.gemv_dev(h, xd.data_ptr(), y_ref.data_ptr())
                be.synchronize()
                free_before = torch.cuda.mem_get_info()[0]
                be.gemv_static_dev(h, xd.data_ptr(), y_new.data_ptr())
                be.synchronize()
                if call == 1:   # the first call on a device may load the kernel's module; the second allocates nothing
                    assert torch.cuda.mem_get_info()[0] == free_before, (m, k)
                want = y_ref.cpu().numpy().view(np.uint16)
                got = y_new.cpu().numpy().view(np.uint16)
                assert rel_l2(got, want) <= 1e-3, (m, k, call)
                # the two entry points may split K differently: equal up to fp32 summation order
                assert np.mean(got == want) > 0.9, (m, k, call)
                cpu = orc.lut_gemv(x, pay, m, k, threads=8)
                assert rel_l2(got, cpu) <= 1e-3 and np.mean(got == cpu) > 0.9, (m, k, call)
            be.free(h)
        # a shape beyond the fixed scratch is refused, not silently allocated for
        big = be.synth("static.big", 64 * 4200, 8192, seed=1)       # K > 4096 forces a split; 4200 row blocks
        xd = torch.zeros(8192, dtype=torch.int16, device="cuda")
        yd = torch.zeros(64 * 4200, dtype=torch.int16, device="cuda")
        torch.cuda.synchronize()
        with pytest.raises(p.PrismCudaError) as e:
            be.gemv_static_dev(big, xd.data_ptr(), yd.data_ptr())
        assert e.value.code == -2 and "fixed scratch" in e.value.msg
        be.free(big)
    finally:
        be.close()
