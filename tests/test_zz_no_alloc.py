"""The allocation-free MLE evaluation (zkh_gl_mle_eval_static) against the regular entry point.

Some callers cannot allocate device memory: a proving service that reserved all of HBM for
its own arena, code between stream-capture begin and end, a loop where an allocation's
device-wide synchronisation is unaffordable.  For them the library keeps its scratch in a
fixed device array.  This file is collected last, so a failure here cannot hide another test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_entry_point_matches_regular_one(orc, zk, prover):
    import torch
    y_dev = torch.zeros(1, dtype=torch.int64, device="cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row through the shared array; the second is smaller, so stale table
    # entries and stale partials from the first are still in the array while it runs
    for v, seed in [(20, 901), (9, 902), (0, 903), (1, 904), (28 if torch.cuda.mem_get_info()[0] > (6 << 30) else 24, 905)]:
        z, s = orc.lcg(v, seed)
        c, _ = orc.lcg(1 << v, s)
        c_dev = zk.p3.to_device(c)
        zk.p3.eval_h_static(c_dev, z, y_dev, stream)
        torch.cuda.synchronize()
        got = int(zk.p3.to_host(y_dev)[0])
        want = prover.eval_h_gpu(c_dev, z)          # existing entry point (bit-exact integer work)
        assert got == want
        if v <= 20:
            assert got == orc.mle_eval(c, z)
        del c_dev


def test_static_entry_point_takes_no_device_memory(orc, zk):
    """After its first call on the device, a call leaves the driver's free-memory figure where it was."""
    import torch
    y_dev = torch.zeros(1, dtype=torch.int64, device="cuda:0")
    z, s = orc.lcg(16, 77)
    c_dev = zk.p3.to_device(orc.lcg(1 << 16, s)[0])
    stream = torch.cuda.current_stream().cuda_stream
    zk.p3.eval_h_static(c_dev, z, y_dev, stream)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        zk.p3.eval_h_static(c_dev, z, y_dev, stream)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0


def test_static_entry_point_rejects_oversize(zk):
    import torch
    y_dev = torch.zeros(1, dtype=torch.int64, device="cuda:0")
    c_dev = torch.zeros(4, dtype=torch.int64, device="cuda:0")
    with pytest.raises(zk.ZkhError) as ei:
        zk.p3.eval_h_static(c_dev, np.zeros(29, dtype=np.uint64), y_dev)
    assert ei.value.code == -5 and "28 variables" in str(ei.value)
    with pytest.raises(zk.ZkhError):
        zk.p3.eval_h_static(c_dev, np.array([0xFFFFFFFF00000001, 0], dtype=np.uint64), y_dev)
