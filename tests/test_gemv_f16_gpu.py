"""f16 weights (WeightFormat::F16): the GEMV over row-major binary16 weights, directly and through a
session with parameter_f16, against numpy (weights rounded to f16 exactly like half::f16::from_f32,
f64 accumulation).  Bar: relative L2 <= 1e-4 per output row."""
import numpy as np
import pytest

from oracle import oracle as O
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,k,n", [(1, 576, 1536), (1, 4096, 4096), (2, 1536, 576), (5, 576, 49152), (2, 320, 100000), (1, 100, 8), (16, 320, 264)])
def test_gemv_f16_matches_numpy(m, k, n):
    import torch
    from meganeura_b200._lib import check, lib
    rng = np.random.Generator(np.random.PCG64(k + n + m))
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    w16 = np.empty((k, n), dtype=np.uint16)
    check(lib.mgq_convert_f16(w.ctypes.data, w.size, w16.ctypes.data))
    assert np.array_equal(w16, w.astype(np.float16).view(np.uint16))          # IEEE round to nearest even
    addend = rng.standard_normal((m, n)).astype(np.float32) if n % 3 == 0 else None
    xd, wd = to_dev(x), to_dev(w16)
    ad = to_dev(addend) if addend is not None else None
    y = torch.full((m, n), 7.0, dtype=torch.float32, device="cuda")
    check(lib.mgq_gemv_f16(xd.data_ptr(), wd.data_ptr(), ad.data_ptr() if ad is not None else None, y.data_ptr(), m, k, n,
                           torch.cuda.current_stream().cuda_stream))
    want = x.astype(np.float64) @ w16.view(np.float16).astype(np.float64)
    if addend is not None:
        want = want + addend
    got = y.cpu().numpy()
    for r in range(m):
        assert O.rel_l2(got[r], want[r]) <= 1e-4


def test_f16_parameter_through_a_session():
    import meganeura_b200 as mg
    g = mg.Graph()
    a = g.input("a", [1, 576])
    w = g.parameter_f16("w", [576, 1536])
    r = g.input("r", [1, 1536])
    g.set_outputs([g.add(g.matmul(a, w), r)])
    s = mg.build_inference_session(g)
    d = s.plan().dispatches
    assert len(d) == 1 and d[0].shader == mg.ShaderEntry.MatMulGemvAdd and d[0].weight_format == mg.WeightFormat.F16
    rng = np.random.Generator(np.random.PCG64(3))
    x = rng.standard_normal((1, 576)).astype(np.float32)
    wf = (rng.standard_normal((576, 1536)) * 0.1).astype(np.float32)
    res = rng.standard_normal((1, 1536)).astype(np.float32)
    s.set_parameter("w", wf)
    s.set_input("a", x)
    s.set_input("r", res)
    s.step()
    s.wait()
    want = x.astype(np.float64) @ wf.astype(np.float16).astype(np.float64) + res
    assert O.rel_l2(s.read_output(1536), want.reshape(-1)) <= 1e-4


def test_f16_shapes_that_are_refused():
    import meganeura_b200 as mg
    from meganeura_b200._lib import check, lib
    import torch
    buf = torch.zeros(4096, dtype=torch.float32, device="cuda")
    with pytest.raises(mg.MgqError):
        check(lib.mgq_gemv_f16(buf.data_ptr(), buf.data_ptr(), None, buf.data_ptr(), 1, 64, 12, None))     # N % 8 != 0
    with pytest.raises(mg.MgqError):
        check(lib.mgq_gemv_f16(buf.data_ptr(), buf.data_ptr(), None, buf.data_ptr(), 17, 64, 16, None))    # more than 16 rows
    g = mg.Graph()
    g.set_outputs([g.matmul(g.input("a", [32, 64]), g.parameter_f16("w", [64, 64]))])
    with pytest.raises(mg.MgqError):
        mg.build_inference_session(g)                                                                       # 32 rows
