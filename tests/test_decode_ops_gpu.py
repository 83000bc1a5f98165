"""The decode-step operators through the C ABI against the numpy restatement of the reference
shaders (oracle/decode_oracle.py).  Tolerances: these are f32 kernels compared with f64 math, so
1e-5 relative to the largest output magnitude unless stated."""
import numpy as np
import pytest

from oracle import decode_oracle as D
from gpu_util import to_dev

pytestmark = pytest.mark.gpu
O_FMT_Q4, O_FMT_Q8 = 2, 3


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def _close(got, want, tol=1e-5):
    want = np.asarray(want, dtype=np.float64)
    err = np.abs(np.asarray(got, dtype=np.float64) - want).max()
    assert err <= tol * max(1.0, np.abs(want).max()), f"max abs err {err:.3e}"


def test_embedding_rows():
    import torch
    from meganeura_b200._lib import check, lib
    rng = np.random.Generator(np.random.PCG64(1))
    table = rng.standard_normal((300, 576)).astype(np.float32)
    ids = np.array([0, 299, 17, 17], dtype=np.uint32)
    out = torch.zeros((4, 576), dtype=torch.float32, device="cuda")
    ids_d, table_d = to_dev(ids), to_dev(table)                       # device inputs must outlive the launch
    check(lib.mgq_embedding(ids_d.data_ptr(), table_d.data_ptr(), out.data_ptr(), 4, 576, 300, _stream()))
    assert np.array_equal(out.cpu().numpy(), D.embedding(ids, table))


@pytest.mark.parametrize("rows,cols,eps", [(1, 576, 1e-5), (1, 4096, 1e-6), (3, 1536, 1e-5), (1, 12288, 1e-6), (2, 20480, 1e-6)])
def test_rms_norm(rows, cols, eps):
    import torch
    from meganeura_b200._lib import check, lib
    rng = np.random.Generator(np.random.PCG64(2))
    x = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
    w = rng.standard_normal(cols).astype(np.float32)
    out = torch.zeros((rows, cols), dtype=torch.float32, device="cuda")
    xd, wd = to_dev(x), to_dev(w)
    check(lib.mgq_rms_norm(xd.data_ptr(), wd.data_ptr(), out.data_ptr(), rows, cols, eps, _stream()))
    _close(out.cpu().numpy(), D.rms_norm(x, w, eps))


@pytest.mark.parametrize("dim,head_dim,theta,pos", [(576, 64, 1e4, 0), (576, 64, 1e4, 383), (4096, 128, 1e6, 2047), (1024, 128, 1e6, 5)])
def test_rope_dynamic(dim, head_dim, theta, pos):
    import torch
    from meganeura_b200._lib import check, lib
    rng = np.random.Generator(np.random.PCG64(3))
    x = rng.standard_normal((1, dim)).astype(np.float32)
    out = torch.zeros((1, dim), dtype=torch.float32, device="cuda")
    xd, posd = to_dev(x), to_dev(np.array([pos], dtype=np.uint32))
    check(lib.mgq_rope_dynamic(xd.data_ptr(), out.data_ptr(), posd.data_ptr(), 1, dim, head_dim, theta, _stream()))
    # angles reach thousands of radians; f32 angle rounding (2^-13 at 2047) bounds the agreement
    _close(out.cpu().numpy(), D.rope(x, theta, pos, head_dim), tol=2e-4 if pos > 100 else 1e-5)


def test_cache_write_touches_one_row():
    import torch
    from meganeura_b200._lib import check, lib
    cache = torch.full((8, 192), 7.0, dtype=torch.float32, device="cuda")
    src = to_dev(np.arange(192, dtype=np.float32).reshape(1, 192))
    pos5, pos8 = to_dev(np.array([5], dtype=np.uint32)), to_dev(np.array([8], dtype=np.uint32))
    check(lib.mgq_cache_write(src.data_ptr(), cache.data_ptr(), pos5.data_ptr(), 192, 8, _stream()))
    host = cache.cpu().numpy()
    assert np.array_equal(host[5], np.arange(192, dtype=np.float32))
    assert (np.delete(host, 5, axis=0) == 7.0).all()
    # a position past the end of the cache writes nothing
    check(lib.mgq_cache_write(src.data_ptr(), cache.data_ptr(), pos8.data_ptr(), 192, 8, _stream()))
    assert np.array_equal(cache.cpu().numpy(), host)


def test_swiglu_separate_and_concatenated():
    import torch
    from meganeura_b200._lib import check, lib
    rng = np.random.Generator(np.random.PCG64(5))
    both = (rng.standard_normal((2, 2 * 1536)) * 4).astype(np.float32)
    dev = to_dev(both)
    out = torch.zeros((2, 1536), dtype=torch.float32, device="cuda")
    check(lib.mgq_swiglu(dev.data_ptr(), dev.data_ptr() + 1536 * 4, out.data_ptr(), 2, 1536, 3072, _stream()))
    _close(out.cpu().numpy(), D.swiglu(both[:, :1536], both[:, 1536:]))
    gate, up = to_dev(both[:1, :1536].copy()), to_dev(both[:1, 1536:].copy())
    check(lib.mgq_swiglu(gate.data_ptr(), up.data_ptr(), out.data_ptr(), 1, 1536, 1536, _stream()))
    _close(out.cpu().numpy()[:1], D.swiglu(both[:1, :1536], both[:1, 1536:]))


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(9, 3, 64), (32, 8, 128), (4, 4, 64), (8, 1, 128)])
@pytest.mark.parametrize("max_seq,pos", [(384, 0), (384, 6), (384, 63), (384, 64), (384, 383), (2048, 1000), (2048, 2047)])
def test_cached_attention(heads, kv_heads, head_dim, max_seq, pos):
    import torch
    from meganeura_b200._lib import check, lib
    rng = np.random.Generator(np.random.PCG64(heads * 1000 + pos))
    kv_dim = kv_heads * head_dim
    q = rng.standard_normal((1, heads * head_dim)).astype(np.float32)
    kc = np.zeros((max_seq, kv_dim), dtype=np.float32)
    vc = np.zeros((max_seq, kv_dim), dtype=np.float32)
    kc[:pos + 1] = rng.standard_normal((pos + 1, kv_dim)).astype(np.float32)
    vc[:pos + 1] = rng.standard_normal((pos + 1, kv_dim)).astype(np.float32)
    kc[pos + 1:] = 1e30                                  # rows past kv_pos must not be read into the result
    ws = torch.zeros(lib.mgq_cached_attention_workspace(kv_heads, head_dim, max_seq), dtype=torch.uint8, device="cuda")
    out = torch.zeros((1, heads * head_dim), dtype=torch.float32, device="cuda")
    posd = to_dev(np.array([pos], dtype=np.uint32))
    qd, kd, vd = to_dev(q), to_dev(kc), to_dev(vc)
    want = D.cached_attention(q, kc, vc, pos, heads, kv_heads, head_dim)
    for _ in range(2):                                   # the workspace returns to its initial state
        out.zero_()
        check(lib.mgq_cached_attention(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), posd.data_ptr(), out.data_ptr(),
                                       heads, kv_heads, head_dim, max_seq, ws.data_ptr(), _stream()))
        _close(out.cpu().numpy(), want, tol=2e-5)


def test_cached_attention_rejects_unbuilt_shapes():
    import torch
    from meganeura_b200 import MgqError
    from meganeura_b200._lib import check, lib
    buf = torch.zeros(4096, dtype=torch.float32, device="cuda")
    p = buf.data_ptr()
    with pytest.raises(MgqError):
        check(lib.mgq_cached_attention(p, p, p, p, p, 4, 2, 96, 16, p, _stream()))      # head_dim 96
    with pytest.raises(MgqError):
        check(lib.mgq_cached_attention(p, p, p, p, p, 18, 2, 64, 16, p, _stream()))     # 9 query heads per KV head
    with pytest.raises(MgqError):
        check(lib.mgq_cached_attention(p, p, p, p, p, 4, 2, 64, 16, None, _stream()))   # no workspace


def test_argmax_lowest_index_wins_and_feedback():
    import torch
    from meganeura_b200._lib import check, lib
    rng = np.random.Generator(np.random.PCG64(9))
    logits = rng.standard_normal(151936).astype(np.float32)
    logits[[70000, 1234, 150000]] = 9.5                  # a three-way tie
    ws = torch.zeros(lib.mgq_argmax_workspace(), dtype=torch.uint8, device="cuda")
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    nxt = torch.zeros(1, dtype=torch.int32, device="cuda")
    pos = to_dev(np.array([3], dtype=np.uint32))
    hist = torch.zeros(8, dtype=torch.int32, device="cuda")
    ld = to_dev(logits)
    for rep in range(2):
        check(lib.mgq_argmax(ld.data_ptr(), logits.size, ws.data_ptr(), tok.data_ptr(), nxt.data_ptr(), pos.data_ptr(),
                             hist.data_ptr(), 8, _stream()))
        assert int(tok.item()) == 1234 == int(np.argmax(logits)) and int(nxt.item()) == 1234
        assert int(pos.cpu().numpy()[0]) == 4 + rep and int(hist[3 + rep].item()) == 1234
    # without feedback nothing but the token is written
    check(lib.mgq_argmax(ld.data_ptr(), 1000, ws.data_ptr(), tok.data_ptr(), None, None, None, 0, _stream()))
    assert int(tok.item()) == int(np.argmax(logits[:1000])) and int(pos.cpu().numpy()[0]) == 5
