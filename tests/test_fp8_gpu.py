"""fp8 (e4m3) block-scaled GEMM and its quantisers against plain PyTorch fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dequant_rows(q, s):
    return q.float() * s.repeat_interleave(128, 1)


def _dequant_blocks(q, s):
    rows, cols = q.shape
    return q.float() * s.repeat_interleave(128, 0)[:rows].repeat_interleave(128, 1)[:, :cols]


def test_quantisers_round_trip():
    from cai_b200 import ops
    torch.manual_seed(0)
    x = (torch.randn(300, 512, device="cuda") * torch.rand(300, 1, device="cuda") * 8).to(torch.bfloat16)
    q, s = ops.quant_rows_1x128(x)
    amax = x.float().view(300, 4, 128).abs().amax(-1)
    assert torch.allclose(s, amax / 448, rtol=1e-6)
    back = _dequant_rows(q, s)
    assert ((back - x.float()).abs() <= 0.07 * amax.repeat_interleave(128, 1) + 1e-6).all()   # e4m3: 3 mantissa bits
    w = torch.randn(384, 200, device="cuda").to(torch.bfloat16)
    qw, sw, qt, st = ops.quant_blocks_128x128(w, transposed=True)
    assert sw.shape == (3, 2) and st.shape == (2, 3) and torch.equal(st, sw.t().contiguous())
    assert torch.equal(qt.view(torch.uint8), qw.view(torch.uint8).t().contiguous())
    backw = _dequant_blocks(qw, sw)
    assert (backw - w.float()).abs().max() <= 0.07 * w.float().abs().max()


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 1024), (200, 264, 384), (1024, 4096, 2048)])
def test_gemm_matches_dequantised_reference(M, N, K):
    from cai_b200 import ops
    torch.manual_seed(1)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    xq, sx = ops.quant_rows_1x128(x)
    wq, sw = ops.quant_blocks_128x128(w)
    ref = _dequant_rows(xq, sx) @ _dequant_blocks(wq, sw).t()     # exactly what the kernel computes, in fp32
    out32 = ops.gemm_fp8(xq, sx, wq, sw, out_dtype=torch.float32)
    assert torch.allclose(out32, ref, atol=1e-3 * ref.abs().max().item(), rtol=1e-3)
    res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    out16 = ops.gemm_fp8(xq, sx, wq, sw, residual=res)
    assert torch.allclose(out16.float(), ref + res.float(), atol=2e-2 * ref.abs().max().item(), rtol=2e-2)
    # against the unquantised product the error is the e4m3 rounding of both operands
    full = x.float() @ w.float().t()
    rel = ((out32 - full).norm() / full.norm()).item()
    assert rel < 0.08, rel
    from cai_b200.ops import _lib
    assert _lib.device_status(clear=True) == 0


def test_training_with_fp8_linear_layers_tracks_bf16():
    """param_dtype = fp8e4m3: forward and input-gradient GEMMs of the linear layers run in e4m3 with
    block scales. The loss curve must stay within a few percent of the bf16 run and fall the same way."""
    from pathlib import Path
    from cai_b200.runtime.engine import Engine, synthetic_batch
    text = (Path(__file__).resolve().parent.parent / "configs" / "tiny.cfg").read_text()
    curves = {}
    for dt in ("bf16", "fp8e4m3"):
        eng = Engine(config_text=text.replace("param_dtype   = bf16", f"param_dtype   = {dt}"), rank=0, world=1, local_rank=0)
        m = eng.model
        rows = eng.hdr.num_microbatches * m.microbatch
        tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows, step=0, seed=9)
        curves[dt] = [eng.step(tok, tgt) for _ in range(8)]
        kernels = {int(x.kernel) for x in eng.plan.exec}
        eng.close()
        if dt == "fp8e4m3":
            from cai_b200 import plan as planlib
            assert planlib.K_GEMM_FP8 in kernels and planlib.K_QUANT_FP8 in kernels
    a, b = curves["bf16"], curves["fp8e4m3"]
    assert b[-1] < b[0] - 0.3, b
    for x, y in zip(a, b):
        assert abs(x - y) < 0.03 * max(1.0, x), (a, b)
