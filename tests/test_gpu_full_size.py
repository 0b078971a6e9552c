"""Parity at the benchmark's own sizes: the decode (c2) and prefill (c3) workloads of bench.py, unfused and fused,
checked on the experts whose weights the bench keeps on the host (experts 0 and 1): every routed row of those
experts against the oracle, and the size-independent properties on all experts (rows past counts[e] untouched,
fused == unfused bytes, scale slop benign)."""
import numpy as np
import pytest
import torch

from oracle import paired_nvfp4_oracle as orc

pytestmark = pytest.mark.gpu

REL_FROB_TOL = 5e-3


def _bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _expert_sf(sfb, e, rows, k):
    per = orc.sf_numel(rows, k, 1)
    return sfb[e * per:(e + 1) * per].cpu().numpy()


@pytest.mark.parametrize("name", ["c2", "c3"])
def test_benchmark_workload_matches_oracle(name):
    import bench
    import paired_nvfp4_kernels  # noqa: F401
    ops = torch.ops.paired_nvfp4
    wl = bench.WORKLOADS[name]
    dev = torch.device("cuda", 0)
    layer = bench.Layer(wl, dev, copies=1, fused=False)
    inputs, counts = bench.make_activation_inputs(wl, layer, 0, 1, dev)
    stream = torch.cuda.current_stream().cuda_stream
    bench.calibrate_second_scale(layer, inputs, stream)
    layer.out1.fill_(-7.0)
    layer.out2.fill_(-7.0)
    layer.step(stream)
    torch.cuda.synchronize()
    E, H, I, cap = layer.E, layer.H, layer.I, layer.cap
    cnt = np.asarray(counts)
    # rows at or past counts[e] keep the caller's bytes, on every expert
    live = torch.arange(cap, device=dev)[None, :] < inputs["counts"][:, None]
    assert bool((layer.out1[~live] == -7.0).all()) and bool((layer.out2[~live] == -7.0).all())
    g1, g2 = inputs["g1"].cpu().numpy(), layer.g2.cpu().numpy()
    b1 = layer.b1[:E * cap].view(E, cap, H // 2)
    for e, (p13, s13, p2, s2) in layer.host_sample.items():
        n = int(cnt[e])
        if n == 0:
            continue
        one = np.array([n], np.int32)
        # GEMM1: the device's own quantized activations through the oracle's dequantised matmul
        want1 = orc.group_mm(orc.dequantize_weight(p13, s13), b1[e:e + 1].cpu().numpy(), _expert_sf(layer.sfb1, e, cap, H),
                             np.array([1.0 / g1[e]], np.float32), one)[0, :n]
        got1 = layer.out1[e, :n].float().cpu().numpy()
        assert orc.rel_frobenius(got1, want1) <= REL_FROB_TOL
        # second quantizer: oracle tail on the device's activation bits, bit for bit
        act = ops.gated_act(layer.out1[e:e + 1], False)
        ob, valid, osfb, _ = orc.silu_mul_quant_act(_bits(layer.out1[e:e + 1]), np.array([g2[e]], np.float32), one,
                                                    act_bits=_bits(act))
        assert np.array_equal(layer.b2[e:e + 1].cpu().numpy()[valid], ob[valid])
        assert np.array_equal(_expert_sf(layer.sfb2, e, cap, I), osfb)
        # GEMM2
        want2 = orc.group_mm(orc.dequantize_weight(p2, s2), layer.b2[e:e + 1].cpu().numpy(), _expert_sf(layer.sfb2, e, cap, I),
                             np.array([1.0 / g2[e]], np.float32), one)[0, :n]
        got2 = layer.out2[e, :n].float().cpu().numpy()
        assert orc.rel_frobenius(got2, want2) <= REL_FROB_TOL
    # fused gate_up epilogue == unfused chain, on every expert: needs the interleaved weight layout
    fl = bench.Layer(wl, dev, copies=1, fused=True)
    fl.set_inputs(g2=layer.g2, a2=layer.al2, **inputs)
    fl.fused = False
    fl.step(stream)                                     # unfused chain on the interleaved weights ...
    torch.cuda.synchronize()
    y = ops.gated_act(fl.out1, True)
    ref_b2, ref_sfb2 = ops.quant_act(y, fl.g2, fl.counts, H)      # ... is gated_act(interleaved) -> quant_act
    fl.fused = True
    fl.b2.zero_()
    fl.step(stream)
    torch.cuda.synchronize()
    assert torch.equal(fl.sfb2, ref_sfb2)
    assert torch.equal(fl.b2[live], ref_b2[live])
