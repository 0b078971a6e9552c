"""Parity at the benchmark's own sizes: the decode (c2), prefill (c3), expert-parallel per-rank (c4r8) and skewed
(c5) workloads of bench.py.  On the experts whose weights the bench keeps on the host (experts 0 and 1) every
routed row is checked against the oracle, expert by expert; on all experts the size-independent properties hold
(rows past counts[e] untouched, fused == unfused bytes, scale slop benign).  c5 is also captured in one CUDA
graph at full size and replayed with fresh Zipf routing (interleaved layout, SiTU with beta = 1.702 and
linear_beta = 1.0), fused and unfused."""
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


@pytest.mark.parametrize("name", ["c2", "c3", "c4r8", "c5"])
def test_benchmark_workload_matches_oracle(name):
    import bench
    import paired_nvfp4_kernels  # noqa: F401
    ops = torch.ops.paired_nvfp4
    wl = bench.WORKLOADS[name]
    dev = torch.device("cuda", 0)
    layer = bench.Layer(wl, dev, copies=1, fused=False)
    inputs, counts = bench.make_activation_inputs(wl, layer, dev)
    stream = torch.cuda.current_stream().cuda_stream
    bench.calibrate_second_scale(layer, inputs, stream)
    layer.out1.fill_(-7.0)
    layer.out2.fill_(-7.0)
    layer.step(stream)
    torch.cuda.synchronize()
    E, H, I, cap = layer.E, layer.H, layer.I, layer.cap
    cnt = np.asarray(counts)
    dev_counts = layer.counts_dev if layer.routed else inputs["counts"]
    assert np.array_equal(dev_counts.cpu().numpy(), cnt)
    # rows at or past counts[e] keep the caller's bytes, on every expert
    live = torch.arange(cap, device=dev)[None, :] < dev_counts[:, None]
    assert bool((layer.out1[~live] == -7.0).all()) and bool((layer.out2[~live] == -7.0).all())
    g1, g2 = inputs["g1"].cpu().numpy(), layer.g2.cpu().numpy()
    b1 = layer.b1[:E * cap].view(E, cap, H // 2)
    checked = 0
    for e, (p13, s13, p2, s2) in layer.host_sample.items():
        n = int(cnt[e])
        if n == 0:
            continue
        checked += 1
        one = np.array([n], np.int32)
        # GEMM1: the device's own quantized activations through the oracle's dequantised matmul
        want1 = orc.group_mm(orc.dequantize_weight(p13, s13), b1[e:e + 1].cpu().numpy(), _expert_sf(layer.sfb1, e, cap, H),
                             np.array([1.0 / g1[e]], np.float32), one)[0, :n]
        got1 = layer.out1[e, :n].float().cpu().numpy()
        assert orc.rel_frobenius(got1, want1) <= REL_FROB_TOL, f"expert {e} gate_up"
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
        assert orc.rel_frobenius(got2, want2) <= REL_FROB_TOL, f"expert {e} down"
    assert checked >= 1 or name == "c5"     # skewed routing may leave experts 0 and 1 empty
    if layer.routed:
        # the combine: every token's kept rows, weighted, in top-k order
        want = orc.moe_finalize(_bits(layer.out2.view(E * cap, H)), layer.route_dest.view(-1, wl["topk"]).cpu().numpy(),
                                layer.router_w.cpu().numpy())
        assert np.array_equal(_bits(layer.final), want)
    g2_t, al2_t = layer.g2, layer.al2
    del layer
    torch.cuda.empty_cache()
    # fused gate_up epilogue == unfused chain, on every expert: needs the interleaved weight layout
    fl = bench.Layer(wl, dev, copies=1, fused=True)
    fl.set_inputs(g2=g2_t, a2=al2_t, **inputs)
    fl.fused = False
    fl.step(stream)                                     # unfused chain on the interleaved weights ...
    torch.cuda.synchronize()
    y = ops.gated_act(fl.out1, True)
    fcounts = fl.counts_dev if fl.routed else fl.counts
    ref_b2, ref_sfb2 = ops.quant_act(y, fl.g2, fcounts, H)      # ... is gated_act(interleaved) -> quant_act
    fl.fused = True
    fl.b2.zero_()
    fl.step(stream)
    torch.cuda.synchronize()
    from paired_nvfp4_kernels import ops as pyops
    assert pyops.group_mm_device_status() == 0
    assert torch.equal(fl.sfb2, ref_sfb2)
    assert torch.equal(fl.b2[live], ref_b2[live])


def test_skewed_workload_replays_in_one_graph_at_full_size():
    import bench
    import paired_nvfp4_kernels  # noqa: F401
    ops = torch.ops.paired_nvfp4
    wl = bench.WORKLOADS["c5"]
    dev = torch.device("cuda", 0)
    E, H, I, cap, T, topk = wl["E"], wl["hidden"], wl["inter"], wl["cap"], wl["tokens"], wl["topk"]
    w, _ = bench.make_expert_weights(wl, dev, range(E), copy=0, fused=True)     # interleaved gate / up rows
    ones = torch.ones(E, device=dev)

    def routing(seed):
        ids, rw = bench.topk_ids(wl, T, E, seed)
        g = torch.Generator(device=dev).manual_seed(seed)
        x = torch.randn((T, H), generator=g, device=dev).to(torch.bfloat16)
        return x, torch.from_numpy(ids).to(dev), torch.from_numpy(rw).to(dev)

    def forward(x, ids, rw, out, fused):
        counts, route_dest, src_tok, src_route = ops.dispatch_plan(ids, 0, E, cap)
        b1, sfb1 = ops.scatter_quant_act_planned(x, src_tok, src_route, None, ones, counts, cap)
        if fused:
            b2, sfb2 = ops.group_mm_swiglu_quant(w["a13"], w["e13"], w["s13"], b1, sfb1, ones, counts, ones, 2 * I, H, 3, 2, 1,
                                                 "situ", 1.702, 1.0)
        else:
            h = torch.empty((E, cap, 2 * I), dtype=torch.bfloat16, device=dev)
            ops.group_mm(h, w["a13"], w["e13"], w["s13"], b1, sfb1, ones, counts, 2 * I, H, 0, 2, 1)
            b2, sfb2 = ops.silu_mul_quant_act(h, ones, counts, H, True, "situ", 1.702, 1.0)
        y = torch.empty((E, cap, H), dtype=torch.bfloat16, device=dev)
        ops.group_mm(y, w["a2"], w["e2"], w["s2"], b2, sfb2, ones, counts, H, I, 0, 2, 1)
        ops.moe_finalize(out, y, route_dest, rw)
        return counts

    x, ids, rw = routing(11)
    x_s, ids_s, rw_s = x.clone(), ids.clone(), rw.clone()          # static inputs of the graphs
    results = {}
    for fused in (True, False):
        out = torch.zeros((T, H), dtype=torch.bfloat16, device=dev)
        forward(x_s, ids_s, rw_s, out, fused)                       # warm up outside capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            counts_g = forward(x_s, ids_s, rw_s, out, fused)
        for seed in (12, 13):
            xn, idn, rwn = routing(seed)
            x_s.copy_(xn), ids_s.copy_(idn), rw_s.copy_(rwn)
            graph.replay()
            torch.cuda.synchronize()
            eager = torch.zeros_like(out)
            counts_e = forward(xn, idn, rwn, eager, fused)
            torch.cuda.synchronize()
            c = counts_e.cpu().numpy()
            assert torch.equal(counts_g, counts_e)
            assert (c == 0).any() and (c == cap).any(), "the skewed routing is meant to leave empty and overflowing experts"
            assert torch.equal(out, eager)
            results[(fused, seed)] = out.clone()
        del graph
    for seed in (12, 13):
        assert torch.equal(results[(True, seed)], results[(False, seed)])       # fused == unfused through the whole layer
    from paired_nvfp4_kernels import ops as pyops
    assert pyops.group_mm_device_status() == 0
