"""GPU: the stream-ordered copy entries, alone and pipelined around a GEMM the way bench.py's
end-to-end arm uses them (upload, product and download on three streams)."""
import ctypes

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


def test_async_copies_round_trip_and_reject_null(gpu):
    import torch
    f = gpu
    lib = f.lib()
    src = torch.arange(1 << 20, dtype=torch.float32).pin_memory()
    dst = torch.empty(1 << 20, dtype=torch.float32).pin_memory()
    dev = torch.empty(1 << 20, device="cuda")
    s = torch.cuda.Stream()
    sp = ctypes.c_void_p(s.cuda_stream)
    assert lib.fastnn_b200_memcpy_h2d_async(_vp(dev), _vp(src), src.numel() * 4, sp) == 0
    assert lib.fastnn_b200_memcpy_d2h_async(_vp(dst), _vp(dev), dst.numel() * 4, sp) == 0
    s.synchronize()
    assert torch.equal(src, dst)
    assert lib.fastnn_b200_memcpy_h2d_async(ctypes.c_void_p(0), _vp(src), 16, sp) == -1
    assert lib.fastnn_b200_memcpy_d2h_async(_vp(dst), ctypes.c_void_p(0), 16, sp) == -1
    assert lib.fastnn_b200_memcpy_h2d_async(ctypes.c_void_p(0), ctypes.c_void_p(0), 0, sp) == 0


def test_pipelined_upload_product_download_matches_the_oracle(gpu):
    import torch
    f = gpu
    lib = f.lib()
    m, n, k = 256, 192, 160
    rng = np.random.default_rng(8)
    hosts = []
    for _ in range(4):
        a = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).pin_memory()
        b = torch.from_numpy(rng.standard_normal((k, n), dtype=np.float32)).pin_memory()
        hosts.append((a, b, torch.empty(m, n, dtype=torch.float32).pin_memory()))
    slots = [(torch.empty(m, k, device="cuda"), torch.empty(k, n, device="cuda"), torch.empty(m, n, device="cuda"))
             for _ in range(2)]
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    for j, (ha, hb, hc) in enumerate(hosts):
        slot = j & 1
        da, db, dc = slots[slot]
        if j >= 2:
            s_in.wait_event(ev_cmp[slot])
        assert lib.fastnn_b200_memcpy_h2d_async(_vp(da), _vp(ha), ha.numel() * 4, ctypes.c_void_p(s_in.cuda_stream)) == 0
        assert lib.fastnn_b200_memcpy_h2d_async(_vp(db), _vp(hb), hb.numel() * 4, ctypes.c_void_p(s_in.cuda_stream)) == 0
        ev_in[slot].record(s_in)
        s_cmp.wait_event(ev_in[slot])
        if j >= 2:
            s_cmp.wait_event(ev_out[slot])
        f.gemm_ex(f.NN, da.data_ptr(), db.data_ptr(), dc.data_ptr(), m, n, k, 1, k, n, n, 0, 0, 0,
                  1.0, 0.0, 0, 0, s_cmp.cuda_stream)
        ev_cmp[slot].record(s_cmp)
        s_out.wait_event(ev_cmp[slot])
        assert lib.fastnn_b200_memcpy_d2h_async(_vp(hc), _vp(dc), hc.numel() * 4, ctypes.c_void_p(s_out.cuda_stream)) == 0
        ev_out[slot].record(s_out)
    s_out.synchronize()
    for ha, hb, hc in hosts:
        want = oracle.matmul(ha.numpy(), hb.numpy())
        err = hc.numpy().astype(np.float64) - want
        assert np.linalg.norm(err) / np.linalg.norm(want) <= 5e-3
    assert f.device_status() == 0
