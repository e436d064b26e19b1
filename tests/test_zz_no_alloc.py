"""The allocation-free InnerProduct entry point, dlp_ip_fwd_enqueue_static.

Some callers of this library may not allocate device memory (they run inside another framework's
memory pool or where cudaMalloc is off limits), so they cannot supply the workspace that
dlp_ip_fwd_enqueue wants; this entry point keeps its scratch in a fixed array inside the library
instead.  The test calls it through the C ABI twice in a row -- with different weights, so a stale
scratch would show -- and compares each result with the regular entry point on the same inputs.
The file sorts last on purpose: if it fails, a run that stops at the first failure has already run
every other test.
"""
import numpy as np
import pytest
import torch

from gpu_util import DEV, REL_TOL, kaiming, rel_err, to_dev

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row():
    from dlprimitives_b200 import capi
    rng = np.random.default_rng(77)
    batch, inputs, outputs = 96, 2048, 1000                 # config 2's InnerProduct shape
    ip = capi.IPForward(inputs, outputs, batch, bias=True, activation="relu")
    assert ip.kernel().startswith("ip_tf32x3")
    ws = torch.empty(max(ip.workspace(), 16), dtype=torch.uint8, device=DEV)
    for call in range(2):
        x = rng.standard_normal((batch, inputs), dtype=np.float32)
        w = kaiming(rng, (outputs, inputs)) * (1.0 + call)   # new weights on the second call
        b = rng.uniform(-0.1, 0.1, outputs).astype(np.float32)
        xd, wd, bd = to_dev(x), to_dev(w), to_dev(b)
        want = torch.full((batch, outputs), float("nan"), device=DEV)
        got = torch.full((batch, outputs), float("nan"), device=DEV)
        ip.enqueue(xd, wd, bd, want, ws)
        ip.enqueue_static(xd, wd, bd, got)
        torch.cuda.synchronize()
        g, r = got.cpu().numpy(), want.cpu().numpy()
        assert not np.isnan(g).any()
        assert rel_err(g, r) <= REL_TOL, (call, rel_err(g, r))
        # the same kernel on the same data; the workspace call may cut K into parts (it has the scratch for
        # the partial sums, this entry point does not), so the two agree to the rounding of the fp32 sum
        assert rel_err(g, r) <= 2e-6
    assert capi.device_status() == 0


def test_static_scratch_refuses_sizes_beyond_its_limit():
    from dlprimitives_b200 import capi
    ip = capi.IPForward(8192, 1024, 4, bias=False)           # packed weights: 64 MiB > 16 MiB
    x = torch.zeros(4, 8192, device=DEV)
    w = torch.zeros(1024, 8192, device=DEV)
    y = torch.zeros(4, 1024, device=DEV)
    with pytest.raises(capi.ValidationError) as e:
        ip.enqueue_static(x, w, None, y)
    assert "static scratch" in str(e.value)
