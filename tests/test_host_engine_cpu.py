"""The host engine runs a GeGLU FFN layer on CPU threads, asynchronously, and agrees with PyTorch."""
import torch
import torch.nn.functional as F

from mesh_b200.runtime.host_engine import HostEngine


def test_ffn_layer_on_the_host_engine():
    torch.manual_seed(0)
    eng = HostEngine(threads=3)
    assert eng.device == "cpu"
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        M, D, Fh = 37, 64, 96
        x = torch.randn(M, D).to(dtype)
        wn = (1 + 0.1 * torch.randn(D)).to(dtype)
        wgu = (torch.randn(2 * Fh, D) / 8).to(dtype)
        wd = (torch.randn(D, Fh) / 8).to(dtype)
        h, gu, act, y, out = (torch.empty(M, n, dtype=dtype) for n in (D, 2 * Fh, Fh, D, D))
        t = eng.submit([("rmsnorm", x, wn, h, 1e-6), ("gemm_nt", h, wgu, gu), ("glu", gu, act, "gelu_tanh"),
                        ("gemm_nt", act, wd, y), ("add", x, y, out)])
        rep = eng.wait(t, 30)
        assert [r["op"] for r in rep] == ["rmsnorm", "gemm_nt", "glu", "gemm_nt", "add"]
        assert all(r["device"] == "cpu" and r["seconds"] > 0 for r in rep)
        xf = x.float()
        hf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wn.float()
        if dtype == torch.bfloat16:
            hf = hf.bfloat16().float()
        guf = hf @ wgu.float().T
        ref = xf + (F.gelu(guf[:, :Fh], approximate="tanh") * guf[:, Fh:]) @ wd.float().T
        assert (out.float() - ref).abs().max() <= tol * ref.abs().max() + tol
    # two batches in flight, waited out of order
    a, b = torch.randn(8, 16), torch.randn(8, 16)
    o1, o2 = torch.empty(8, 16), torch.empty(8, 16)
    t1 = eng.submit([("add", a, b, o1)])
    t2 = eng.submit([("add", o1, b, o2)])
    eng.wait(t2)
    eng.wait(t1)
    assert torch.allclose(o2, a + 2 * b)
    eng.close()
