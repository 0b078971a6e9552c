#!/usr/bin/env python
"""Benchmark of the paired-4:8 sparse NVFP4 grouped MoE GEMM path on B200.

    python bench.py --gpus N --steps K --warmup W [--workload c2|c2b|c3|c4|c4r8|c5] [--impl reference]

A "pass" is one expert-FFN pass of a MoE layer over one batch of synthetic, seeded, model-shaped input.
A "step" is `passes_per_step` passes back to back (chosen so that the K timed steps last at least half a
second, long enough for the clock sampler to see them; the line says how many).

Headline workload (every N, so that a 1-2-4-8 series is one curve): c4, the expert-parallel DeepSeek-V3-shaped
layer - 256 experts sharded over the N ranks, 8192 tokens per rank, top-8.  A pass is the whole layer: slab
plan -> quant_rows -> pack_wire_rows -> all-to-all -> dispatch_plan -> scatter_fp4_wire -> group_mm (gate_up,
fused SwiGLU + quantize) -> zero_rows + group_mm_rows (down, rows straight into return order) -> all-to-all -> moe_finalize, with fresh routing
work inside the pass.  At N = 1 the two all-to-alls are the identity and everything else is the same code.
`value` is dense-equivalent TFLOP/s of the two grouped GEMMs over the kept rows of all ranks, inputs resident
in HBM; `e2e` is the same with the tokens in pinned host memory (copy in, layer, copy out, inside the timed
region).  At N = 1 the line also carries the single-GPU decode (c2) and prefill (c3) workloads under
`workloads`, each with its own kernel times and rooflines, a CPU baseline and, at every N, a per-phase
breakdown and a parity check of the exchanged result against the single-GPU operators.

`--workload X` makes X the (single-GPU) headline instead.  `--impl reference` times the CPU implementation of
the path alone, on bounded samples of the same workload.
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "grouped-sparse-gemm_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

FALLBACK_HBM_GBS = 6650.0      # earlier measurement on this pool, used only without MEASURED_PEAKS.json
# Dense-equivalent rate of the 2:4-sparse FP4 tensor pipe.  No measured figure exists on this pool (the driver
# measures bf16 only), so tensor-bound launches are reported against the nominal 18 PFLOP/s; for scale, one
# 128 x 128 x 128 sparse MMA was measured to hold an SM for 96 cycles, which is 12.7 PFLOP/s over 148 SMs.
NOMINAL_SPARSE_FP4_TFLOPS = 18000.0

# dram__bytes_read.sum + dram__bytes_write.sum of one gate_up group_mm launch, from the ncu captures summarised
# under profiles/ (c2, c3: the same workload; c4: a capture of 32 of the 256 experts with the same rows per expert,
# times 8 - the traffic is the weights and rows of the experts, so it grows with their number); None where no
# capture exists
NCU_TRAFFIC_BYTES = {"c2": 331.3e6, "c3": 336.5e6, "c4": 8 * 376.2e6}

WORKLOADS = {
    # Mixtral-8x7B expert FFN, decode: per-expert counts uniform in [1, 16]
    "c2": dict(desc="decode Mixtral-8x7B-shaped expert FFN", E=8, hidden=4096, inter=14336, cap=16,
               routing="counts", seed=1001, config_id=7, wstd=0.02),
    # one active expert of a 32-expert shard, one token: the decode case of an expert-parallel rank
    "c2b": dict(desc="decode, one active expert of a DeepSeek-V3-shaped 32-expert shard", E=32, hidden=7168, inter=2048,
                cap=16, routing="one", seed=1006, config_id=7, wstd=0.02),
    # Qwen3-30B-A3B MoE, prefill: 16384 tokens, top-8 of 128, cap 2048
    "c3": dict(desc="prefill Qwen3-30B-A3B-shaped MoE", E=128, hidden=2048, inter=768, cap=2048,
               routing="topk", tokens=16384, topk=8, seed=1002, config_id=1, wstd=0.02),
    # DeepSeek-V3 MoE, expert parallel: 8192 tokens per rank, top-8 of 256
    "c4": dict(desc="DeepSeek-V3-shaped MoE, expert parallel", E=256, hidden=7168, inter=2048, cap=1024,
               routing="topk", tokens=8192, topk=8, seed=1003, config_id=1, wstd=0.02),
    # the per-rank shape of c4 at 8 ranks (32 local experts, 65536 routed rows), without the exchange
    "c4r8": dict(desc="DeepSeek-V3-shaped MoE, one rank's expert shard at 8 ranks", E=32, hidden=7168, inter=2048,
                 cap=4096, routing="topk", tokens=8192, topk=8, seed=1005, config_id=1, wstd=0.02),
    # skewed routing: Zipf(1.2) expert popularity, top-4 of 128 over 8192 tokens, cap 4096
    "c5": dict(desc="skewed-routing MoE (Zipf 1.2)", E=128, hidden=3072, inter=3072, cap=4096,
               routing="zipf", tokens=8192, topk=4, seed=1004, config_id=1, wstd=0.02),
}
METRIC = "moe_expert_ffn_group_mm_dense_equiv_tflops"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--config-id", type=int, default=None, help="group_mm tile variant override")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-sub-workloads", action="store_true", help="N = 1: skip the c2 / c3 entries of `workloads`")
    ap.add_argument("--unfused", action="store_true", help="separate silu_mul_quant_act launch instead of the fused GEMM1 epilogue")
    ap.add_argument("--passes", type=int, default=None,
                    help="passes per step (default: as many as make the timed steps last half a second); "
                         "small values keep a profiler capture short")
    ap.add_argument("--experts", type=int, default=None,
                    help="run a routed workload with this many experts and proportionally fewer tokens (the same "
                         "rows per expert): a smaller copy of the workload for profiler captures")
    ap.add_argument("--exchange", default="direct", choices=["direct", "nccl"],
                    help="N > 1: 'direct' = the producing kernels store wire rows and expert outputs straight into the "
                         "other ranks' buffers (peer memory); 'nccl' = an all-to-all either side of the local FFN")
    ap.add_argument("--slab-headroom", type=float, default=1.125, help="expert-parallel slab rows over the mean load")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------
# byte / flop accounting (algorithmic: what the math needs, independent of the implementation)
# ------------------------------------------------------------------------------------------------

def _ru(a, b):
    return -(-a // b) * b


def gemm_bytes(active, M, K, rows, out_bytes_per_row=None):
    """Weights of the active experts (codes + metadata + scales) + activation codes/scales in + output
    (bf16 unless given); the same formula the reference's tools/bench_moe.py uses (sparse_bytes)."""
    kb = -(-K // 32)
    w = active * (M * K // 4 + _ru(M, 128) * _ru(K, 256) // 16 + _ru(M, 128) * _ru(kb, 4))
    return w + rows * (K // 2 + K // 32) + rows * (2 * M if out_bytes_per_row is None else out_bytes_per_row)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def launch_roofline(name, nbytes, flops, seconds, traffic=None):
    """max(bytes / HBM peak, flops / tensor peak) decides the bound; achieved and peak are in that bound's unit."""
    hbm, src = peaks()
    t_hbm, t_tensor = nbytes / (hbm * 1e9), flops / (NOMINAL_SPARSE_FP4_TFLOPS * 1e12)
    if t_hbm >= t_tensor:
        ach = nbytes / seconds / 1e9
        return dict(bound="hbm", kernel=name, achieved=ach, peak=hbm, unit="GB/s", frac=ach / hbm, peak_source=src,
                    traffic=traffic, algorithmic_bytes=nbytes, dense_equiv_flops=flops, launch_us=seconds * 1e6)
    ach = flops / seconds / 1e12
    return dict(bound="tensor", kernel=name, achieved=ach, peak=NOMINAL_SPARSE_FP4_TFLOPS, unit="TFLOP/s",
                frac=ach / NOMINAL_SPARSE_FP4_TFLOPS,
                peak_source="nominal 2:4-sparse FP4 in dense-equivalent flops (no measured FP4 peak on this pool; "
                            "measured MMA issue rate: 12700)",
                traffic=traffic, algorithmic_bytes=nbytes, dense_equiv_flops=flops, launch_us=seconds * 1e6)


def gemm_rooflines(wl_name, H, I, rows, active, fused, t13, t2):
    """Rooflines of the two group_mm launches of a pass: gate_up (M = 2I, K = H) and down (M = H, K = I)."""
    out13 = (I // 2 + I // 32) if fused else None
    r13 = launch_roofline("group_mm gate_up" + (" (fused SwiGLU + quantize)" if fused else ""),
                          gemm_bytes(active, 2 * I, H, rows, out13), 2.0 * rows * 2 * I * H, t13,
                          NCU_TRAFFIC_BYTES.get(wl_name) if fused else None)
    r2 = launch_roofline("group_mm down", gemm_bytes(active, H, I, rows), 2.0 * rows * H * I, t2)
    return r13, r2


# ------------------------------------------------------------------------------------------------
# synthetic inputs
# ------------------------------------------------------------------------------------------------

def topk_ids(wl, tokens, E_total, seed):
    rng = np.random.default_rng(seed)
    logits = rng.standard_normal((tokens, E_total)).astype(np.float32)
    if wl["routing"] == "zipf":
        ranks = rng.permutation(E_total) + 1
        logits += np.log((1.0 / ranks ** 1.2) / np.sum(1.0 / ranks ** 1.2)).astype(np.float32)
    ids = np.argpartition(-logits, wl["topk"] - 1, axis=1)[:, :wl["topk"]]
    order = np.argsort(-np.take_along_axis(logits, ids, 1), axis=1, kind="stable")
    ids = np.take_along_axis(ids, order, 1)
    sel = np.take_along_axis(logits, ids, 1)
    w = np.exp(sel - sel.max(1, keepdims=True))
    w = (w / w.sum(1, keepdims=True)).astype(np.float32)
    return ids.astype(np.int64), w


def expert_counts(ids, first_expert, num_local, cap):
    flat = ids.reshape(-1) - first_expert
    flat = flat[(flat >= 0) & (flat < num_local)]
    return np.minimum(np.bincount(flat, minlength=num_local), cap).astype(np.int32)


def make_expert_weights(wl, device, experts, copy=0, fused=True):
    """Compressed weights of the given global expert ids: N(0, wstd), pruned paired-4:8, NVFP4; generated per
    expert on the GPU with the package's torch weight spec (bit-identical to the reference's reference.py).
    Returns dict(a13, e13, s13, a2, e2, s2) and the packed bytes of the first two experts (host copies)."""
    import torch
    import paired_nvfp4_kernels as pnk
    from paired_nvfp4_kernels import reference as wref
    ops = torch.ops.paired_nvfp4
    H, I = wl["hidden"], wl["inter"]
    perm = pnk.interleave_gate_up_rows(I, device=device) if fused else None
    parts13, parts2, host = [], [], {}
    for i, e in enumerate(experts):
        g = torch.Generator(device=device).manual_seed(wl["seed"] * 7919 + 1000 * copy + int(e))
        w13 = torch.randn((1, 2 * I, H), generator=g, device=device) * wl["wstd"]
        w2 = torch.randn((1, H, I), generator=g, device=device) * wl["wstd"]
        p13, s13, _ = wref.quantize_weight(wref.prune_paired_4of8(w13))
        if fused:   # gate/up rows interleaved in 64-row blocks for the fused epilogue
            p13, s13 = p13[:, perm].contiguous(), s13[:, perm].contiguous()
        p2, s2, _ = wref.quantize_weight(wref.prune_paired_4of8(w2))
        if copy == 0 and i < 2:
            host[i] = tuple(t.cpu().numpy() for t in (p13, s13, p2, s2))
        parts13.append(ops.compress(p13, s13, H))
        parts2.append(ops.compress(p2, s2, I))
        del w13, w2, p13, s13, p2, s2
    cat = lambda parts, i: torch.cat([p[i] for p in parts], 0) if i < 2 else torch.cat([p[i] for p in parts])
    return dict(a13=cat(parts13, 0), e13=cat(parts13, 1), s13=cat(parts13, 2),
                a2=cat(parts2, 0), e2=cat(parts2, 1), s2=cat(parts2, 2)), host


class Layer:
    """Device state of one single-GPU expert-FFN layer and the launches of a pass, through the C ABI.
    Decode workloads: quant_act -> group_mm (gate_up) [-> silu_mul_quant_act] -> group_mm (down).
    Routed workloads: dispatch_plan -> scatter_quant_act_planned -> the same GEMMs -> moe_finalize."""

    PHASES_DECODE = ("quant_act", "group_mm_gate_up", "silu_mul_quant_act", "group_mm_down")
    PHASES_ROUTED = ("dispatch_plan", "scatter_quant_act_planned", "group_mm_gate_up", "silu_mul_quant_act",
                     "group_mm_down", "moe_finalize")

    def __init__(self, wl, device, config_id=None, copies=2, fused=True):
        import torch
        from paired_nvfp4_kernels import _cabi
        self.torch, self.lib, self.cabi = torch, _cabi.lib, _cabi
        self.wl, self.dev = wl, device
        self.E, self.H, self.I, self.cap = wl["E"], wl["hidden"], wl["inter"], wl["cap"]
        self.cfg = wl["config_id"] if config_id is None else config_id
        self.fused = fused
        names = _cabi.group_mm_config_names()
        self.cluster_m = 2 if names[self.cfg].split("_")[1] == "2sm" else 1
        # fused variant with the same tile as the chosen group_mm variant
        self.fused_cfg = {6: 0, 7: 0, 4: 1, 5: 2, 0: 3, 1: 5, 2: 4, 3: 4, 8: 4}[self.cfg]
        self.fused_cluster_m = 2 if _cabi.group_mm_swiglu_config_names()[self.fused_cfg].split("_")[1] == "2sm" else 1
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        E, H, I, cap = self.E, self.H, self.I, self.cap
        self.weights, self.host_sample = [], {}
        for c in range(copies):
            w, host = make_expert_weights(wl, device, range(E), copy=c, fused=fused)
            self.weights.append(w)
            if c == 0:
                self.host_sample = host
        u8 = dict(dtype=torch.uint8, device=device)
        self.b1 = torch.empty((E * cap + 1, H // 2), **u8)
        self.sfb1 = torch.empty((_cabi.sf_numel(cap, H, E),), **u8)
        self.out1 = torch.zeros((E, cap, 2 * I), dtype=torch.bfloat16, device=device)
        self.b2 = torch.empty((E, cap, I // 2), **u8)
        self.sfb2 = torch.empty((_cabi.sf_numel(cap, I, E),), **u8)
        self.out2 = torch.zeros((E, cap, H), dtype=torch.bfloat16, device=device)
        ws13 = int(self.lib.pnv_group_mm_workspace_bytes(E, 2 * I, cap, self.sm_count))
        ws2 = int(self.lib.pnv_group_mm_workspace_bytes(E, H, cap, self.sm_count))
        self.ws_bytes = max(ws13, ws2)
        self.ws = torch.zeros((self.ws_bytes,), **u8) if self.ws_bytes else None      # split-K workspace (decode sizes only)
        self.routed = wl["routing"] in ("topk", "zipf")
        if self.routed:
            T, topk = wl["tokens"], wl["topk"]
            i32 = dict(dtype=torch.int32, device=device)
            self.counts_dev = torch.zeros((E,), **i32)
            self.route_dest = torch.empty((T * topk,), **i32)
            self.src_tok = torch.empty((E * cap,), **i32)
            self.src_route = torch.empty((E * cap,), **i32)
            self.scratch = torch.empty((max(int(self.lib.pnv_dispatch_plan_scratch_ints(T * topk, E)), 1),), **i32)
            self.final = torch.zeros((T, H), dtype=torch.bfloat16, device=device)

    def set_inputs(self, x, counts, g1, a1, g2, a2, ids=None, router_w=None):
        """x: bf16 [E, cap, H] (decode) or [T, H] (routed).  All device tensors."""
        self.x, self.counts, self.g1, self.al1, self.g2, self.al2 = x, counts, g1, a1, g2, a2
        self.ids, self.router_w = ids, router_w

    def phases(self):
        return self.PHASES_ROUTED if self.routed else self.PHASES_DECODE

    def step(self, stream, c=0, events=None):
        """One pass; `events`, when given, holds len(phases()) + 1 CUDA events recorded around the launches."""
        lib, ck = self.lib, self.cabi.check
        w = self.weights[c % len(self.weights)]
        E, H, I, cap, sm = self.E, self.H, self.I, self.cap, self.sm_count
        ws = self.ws.data_ptr() if self.ws is not None else None
        ev = iter(events) if events else None
        mark = (lambda: next(ev).record()) if events else (lambda: None)
        mark()
        if self.routed:
            T, topk = self.ids.shape
            counts = self.counts_dev
            ck(lib.pnv_dispatch_plan(self.ids.data_ptr(), 1, T, topk, 0, E, cap, counts.data_ptr(),
                                     self.route_dest.data_ptr(), self.src_tok.data_ptr(), self.src_route.data_ptr(),
                                     self.scratch.data_ptr(), stream))
            mark()
            ck(lib.pnv_scatter_quant_act_planned(self.x.data_ptr(), self.src_tok.data_ptr(), self.src_route.data_ptr(), None,
                                                 self.g1.data_ptr(), 1, counts.data_ptr(), H, E, cap, self.b1.data_ptr(),
                                                 self.sfb1.data_ptr(), sm, stream))
        else:
            counts = self.counts
            ck(lib.pnv_quant_act(self.x.data_ptr(), self.g1.data_ptr(), 1, counts.data_ptr(), E, cap, H,
                                 self.b1.data_ptr(), self.sfb1.data_ptr(), sm, stream))
        mark()
        if self.fused:
            ck(lib.pnv_group_mm_swiglu_quant(self.b2.data_ptr(), self.sfb2.data_ptr(), w["a13"].data_ptr(),
                                             w["e13"].data_ptr(), w["s13"].data_ptr(), self.b1.data_ptr(),
                                             self.sfb1.data_ptr(), self.al1.data_ptr(), counts.data_ptr(),
                                             self.g2.data_ptr(), 1, E, 2 * I, H, cap, self.fused_cfg, self.fused_cluster_m, 1,
                                             0, 1.0, -1.0, sm, 1, ws, self.ws_bytes, stream))
            mark()
        else:
            ck(lib.pnv_group_mm(self.out1.data_ptr(), w["a13"].data_ptr(), w["e13"].data_ptr(), w["s13"].data_ptr(),
                                self.b1.data_ptr(), self.sfb1.data_ptr(), self.al1.data_ptr(), counts.data_ptr(),
                                E, 2 * I, H, cap, self.cfg, self.cluster_m, 1, sm, 1, ws, self.ws_bytes, stream))
            mark()
            ck(lib.pnv_silu_mul_quant_act(self.out1.data_ptr(), self.g2.data_ptr(), 1, counts.data_ptr(), E, cap,
                                          I, 0, 0, 1.0, -1.0, self.b2.data_ptr(), self.sfb2.data_ptr(), sm, stream))
            mark()
        ck(lib.pnv_group_mm(self.out2.data_ptr(), w["a2"].data_ptr(), w["e2"].data_ptr(), w["s2"].data_ptr(),
                            self.b2.data_ptr(), self.sfb2.data_ptr(), self.al2.data_ptr(), counts.data_ptr(),
                            E, H, I, cap, self.cfg, self.cluster_m, 1, sm, 1, ws, self.ws_bytes, stream))
        mark()
        if self.routed:
            T, topk = self.ids.shape
            ck(lib.pnv_moe_finalize(self.final.data_ptr(), self.out2.data_ptr(), self.route_dest.data_ptr(),
                                    self.router_w.data_ptr(), T, topk, H, stream))
            mark()


def make_activation_inputs(wl, layer, device, seed_shift=0):
    """Seeded activations / routing; returns kwargs for Layer.set_inputs and the host counts."""
    import torch
    E, H, cap = layer.E, layer.H, layer.cap
    seed = wl["seed"] + seed_shift
    g = torch.Generator(device=device).manual_seed(seed)
    ids = router_w = None
    if wl["routing"] in ("counts", "one"):
        if wl["routing"] == "one":
            counts = np.zeros(E, np.int32)
            counts[E // 3] = 1
        else:
            counts = np.random.default_rng(seed).integers(1, cap + 1, E).astype(np.int32)
        x = torch.randn((E, cap, H), generator=g, device=device).to(torch.bfloat16)
        amax = torch.stack([x[e, :max(int(counts[e]), 1)].abs().max() for e in range(E)]).float()
    else:
        T = wl["tokens"]
        ids_np, w = topk_ids(wl, T, wl["E"], seed)
        counts = expert_counts(ids_np, 0, E, cap)
        x = torch.randn((T, H), generator=g, device=device).to(torch.bfloat16)
        amax = x.abs().max().float().expand(E).contiguous()
        ids = torch.from_numpy(ids_np).to(device)
        router_w = torch.from_numpy(w).to(device)
    g1 = (6.0 * 448.0 / amax.clamp(min=1e-6)).contiguous()
    return dict(x=x, counts=torch.from_numpy(counts).to(device), g1=g1, a1=(1.0 / g1).contiguous(), ids=ids,
                router_w=router_w), counts


def calibrate_second_scale(layer, inputs, stream):
    """gscale of the second quantizer from the actual activation range of a warm-up pass."""
    import torch
    E = layer.E
    ones = torch.ones(E, device=layer.dev)
    layer.set_inputs(g2=ones, a2=ones, **inputs)
    was_fused, layer.fused = layer.fused, False
    layer.step(stream)
    torch.cuda.synchronize()
    layer.fused = was_fused
    y = torch.ops.paired_nvfp4.gated_act(layer.out1, was_fused)
    cnt = inputs["counts"].cpu().numpy()
    amax = torch.stack([y[e, :int(cnt[e])].abs().max() if cnt[e] > 0 else torch.ones((), device=layer.dev) for e in range(E)])
    g2 = (6.0 * 448.0 / amax.float().clamp(min=1e-6)).contiguous()
    layer.set_inputs(g2=g2, a2=(1.0 / g2).contiguous(), **inputs)


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        nv = self.nv
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv is not None:
            self.t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self.nv is not None:
            self.t.join(timeout=1.0)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def passes_for(est_pass_s, steps, target_s=0.5, cap=256):
    return int(max(1, min(cap, np.ceil(target_s / max(steps * est_pass_s, 1e-9)))))


# ------------------------------------------------------------------------------------------------
# single-GPU workloads (c2, c2b, c3, c4r8, c5): measured through the C ABI
# ------------------------------------------------------------------------------------------------

def run_local_workload(wl_name, wl, device, args, steps, warmup, sample_clocks=None, with_e2e=True, with_cpu=True):
    """Times `steps` steps of one single-GPU workload.  Returns the fields of a bench line for it."""
    import torch
    import paired_nvfp4_kernels
    fused = not args.unfused
    layer = Layer(wl, device, config_id=args.config_id, fused=fused)
    inputs, counts = make_activation_inputs(wl, layer, device)
    stream = torch.cuda.current_stream().cuda_stream
    calibrate_second_scale(layer, inputs, stream)
    rows, active = int(counts.sum()), int((counts > 0).sum())
    H, I = layer.H, layer.I
    flops = 2.0 * rows * (2 * I * H + H * I)
    names = layer.phases()
    if fused:
        names = tuple(n for n in names if n != "silu_mul_quant_act")

    for i in range(3):
        layer.step(stream, c=i)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(3):
        layer.step(stream, c=i)
    e1.record()
    torch.cuda.synchronize()
    passes = args.passes or passes_for(e0.elapsed_time(e1) / 3 * 1e-3, steps)
    for i in range(warmup * passes):
        layer.step(stream, c=i)
    # every pass carries its phase events; steps are timed as a whole
    phase_evs = [[torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)] for _ in range(steps * passes)]
    step_evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    torch.cuda.synchronize()
    sampler = sample_clocks if sample_clocks is not None else _NullCtx()
    with sampler:
        step_evs[0].record()
        for s in range(steps):
            for p_ in range(passes):
                layer.step(stream, c=s * passes + p_, events=phase_evs[s * passes + p_])
            step_evs[s + 1].record()
        torch.cuda.synchronize()
    step_ms = np.array([step_evs[s].elapsed_time(step_evs[s + 1]) for s in range(steps)])
    ms_step = float(step_evs[0].elapsed_time(step_evs[steps])) / steps
    phase_us = {n: float(np.mean([ev[i].elapsed_time(ev[i + 1]) for ev in phase_evs])) * 1e3 for i, n in enumerate(names)}
    pass_s = ms_step * 1e-3 / passes
    r13, r2 = gemm_rooflines(wl_name, H, I, rows, active, fused, phase_us["group_mm_gate_up"] * 1e-6,
                             phase_us["group_mm_down"] * 1e-6)
    dominant = r13 if r13["launch_us"] >= r2["launch_us"] else r2
    bytes_total = (r13["algorithmic_bytes"] + r2["algorithmic_bytes"] + rows * (2 * H + H // 2 + H // 32)
                   + (0 if fused else rows * (4 * I + I // 2 + I // 32)))
    res = dict(
        value=flops / pass_s / 1e12, ms_per_step=ms_step, passes_per_step=passes, layer_us=pass_s * 1e6,
        step_ms_mean=float(step_ms.mean()), step_ms_p10=float(np.percentile(step_ms, 10)),
        hbm_gbs_layer=bytes_total / pass_s / 1e9, kernels_us=phase_us, roofline=dominant,
        rooflines={"group_mm_gate_up": r13, "group_mm_down": r2},
        config={"workload": f"{wl_name}: {wl['desc']}", "experts": wl["E"], "experts_per_gpu": wl["E"], "hidden": H,
                "intermediate": I, "cap": wl["cap"], "routed_rows": rows, "active_experts": active,
                "tile_config": paired_nvfp4_kernels.group_mm_configs()[layer.cfg],
                "fused_swiglu_epilogue": fused, "passes_per_step": passes,
                "l2": "two weight copies alternate; every pass streams more than the 126 MB L2"},
        # dispatch_plan is three launches for plans of more than 1024 routings
        gpu_launches=(len(names) + (2 if layer.routed else 0)) * passes * steps, flops_per_pass=flops)
    if layer.routed:
        # moe_finalize is HBM bound: every kept row read once, one row written per token
        T = wl["tokens"]
        fin_bytes = rows * 2 * H + T * 2 * H
        res["rooflines"]["moe_finalize"] = launch_roofline("moe_finalize", fin_bytes, 0.0, phase_us["moe_finalize"] * 1e-6)
    if with_e2e and not args.no_e2e:
        res["e2e"] = run_local_e2e(layer, wl, flops, max(5, min(steps * passes, 200)))
    if with_cpu and not args.no_cpu_baseline:
        res["cpu_baseline"] = run_cpu_baseline(layer.host_sample, inputs, counts, layer)
    del layer
    torch.cuda.empty_cache()
    return res


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def run_local_e2e(layer, wl, flops, n):
    """The user's call path: torch.ops.paired_nvfp4.* with freshly allocated outputs; every pass copies the
    activations in from pinned host memory and the layer output back out.  The launches are fixed-shape and read
    counts on the device, so the pass is captured once in a CUDA graph, as a serving loop would, and replayed."""
    import torch
    ops = torch.ops.paired_nvfp4
    x = layer.x
    host_x = x.cpu().pin_memory()
    dev_x = torch.empty_like(x)
    E, H, I, cap = layer.E, layer.H, layer.I, layer.cap
    out1 = torch.zeros((E, cap, 2 * I), dtype=torch.bfloat16, device=x.device)
    out2 = torch.zeros((E, cap, H), dtype=torch.bfloat16, device=x.device)
    w = layer.weights[0]
    name = layer.cabi.group_mm_config_names()[layer.cfg]
    if layer.routed:
        T = layer.ids.size(0)
        final = torch.zeros((T, H), dtype=torch.bfloat16, device=x.device)
        host_out = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
    else:
        final = out2
        host_out = torch.empty((E, cap, H), dtype=torch.bfloat16).pin_memory()

    def one():
        dev_x.copy_(host_x, non_blocking=True)
        if layer.routed:
            counts, route_dest, src_tok, src_route = ops.dispatch_plan(layer.ids, 0, E, cap)
            b1, s1 = ops.scatter_quant_act_planned(dev_x, src_tok, src_route, None, layer.g1, counts, cap)
        else:
            counts = layer.counts
            b1, s1 = ops.quant_act(dev_x, layer.g1, counts, 2 * I)
        if layer.fused:
            b2, s2 = ops.group_mm_swiglu_quant(w["a13"], w["e13"], w["s13"], b1, s1, layer.al1, counts, layer.g2,
                                               2 * I, H, layer.fused_cfg, layer.fused_cluster_m, 1)
        else:
            ops.group_mm(out1, w["a13"], w["e13"], w["s13"], b1, s1, layer.al1, counts, 2 * I, H, layer.cfg,
                         layer.cluster_m, 1)
            b2, s2 = ops.silu_mul_quant_act(out1, layer.g2, counts, H)
        ops.group_mm(out2, w["a2"], w["e2"], w["s2"], b2, s2, layer.al2, counts, H, I, layer.cfg, layer.cluster_m, 1)
        if layer.routed:
            ops.moe_finalize(final, out2, route_dest, layer.router_w)
        host_out.copy_(final, non_blocking=True)

    def eager():
        one()
        torch.cuda.synchronize()

    for _ in range(3):
        eager()
    mode = "cuda graph replay"
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                one()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()

        def run():
            graph.replay()
            torch.cuda.synchronize()
        check = host_out.clone()
        host_out.zero_()
        run()
        assert torch.equal(host_out, check), "graph replay does not reproduce the eager pass"
    except Exception as exc:   # capture unavailable: time the eager calls
        mode = f"eager calls (graph capture failed: {type(exc).__name__})"
        run = eager
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3) / n
    return dict(value=flops / (ms * 1e-3) / 1e12, unit="TFLOP/s", ms_per_pass=ms,
                h2d_bytes_per_step=host_x.numel() * 2, d2h_bytes_per_step=host_out.numel() * 2,
                passes=n, tile_config=name, mode=mode)


# ------------------------------------------------------------------------------------------------
# CPU baseline: the reference's reference.py (weight half, when oracle/_ref holds it) + the numpy oracle
# ------------------------------------------------------------------------------------------------

def load_reference_py():
    """The reference's own paired_nvfp4_kernels/reference.py, placed under oracle/_ref/ by oracle/build_ref.py
    (git-ignored, travels to the GPU box); None when it is not there."""
    path = os.path.join(ROOT, "oracle", "_ref", "reference.py")
    if not os.path.exists(path):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("pnv_reference_py", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def cpu_weight_half(ref, orc, M, K, wstd, seed):
    """prune + quantize one [1, M, K] weight on the host: the reference's reference.py when present."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((1, M, K)) * wstd).astype(np.float32)
    if ref is not None:
        import torch
        torch.set_num_threads(os.cpu_count())
        packed, sf, _ = ref.quantize_weight(ref.prune_paired_4of8(torch.from_numpy(w)))
        return packed.numpy(), sf.view(torch.uint8).numpy()
    packed, sf, _ = orc.quantize_weight(orc.prune_paired_4of8(w))
    return packed, sf


def cpu_layer_pass(orc, sample, x_bits, counts, g1):
    """One expert-FFN pass on the host for the sampled experts: quantize, dequantise the stored
    weights, fp32 matmuls.  Returns dense-equivalent flops done."""
    flops = 0.0
    for e, (p13, s13, p2, s2) in sample.items():
        n = int(counts[e])
        if n == 0:
            continue
        w13 = orc.dequantize_weight(p13, s13)
        w2 = orc.dequantize_weight(p2, s2)
        cnt = np.array([n], np.int32)
        b1, _, sfb1 = orc.quant_act(x_bits[e:e + 1, :n], np.array([g1[e]], np.float32), cnt)
        o1 = orc.group_mm(w13, b1, sfb1, np.array([1.0 / g1[e]], np.float32), cnt)
        o1b = orc.f32_to_bf16_bits(o1)
        b2, _, sfb2, _ = orc.silu_mul_quant_act(o1b, np.ones(1, np.float32), cnt)
        orc.group_mm(w2, b2, sfb2, np.ones(1, np.float32), cnt)
        flops += 2.0 * n * (w13.shape[1] * w13.shape[2] + w2.shape[1] * w2.shape[2])
    return flops


def run_cpu_baseline(host_sample, inputs, counts, layer, budget_s=12.0):
    """Experts 0 and 1 of the workload on the host cores: every routed row of theirs (at most 64 each)."""
    from oracle import paired_nvfp4_oracle as orc
    x = inputs["x"]
    cnt = np.asarray(counts).copy()
    g1 = inputs["g1"].cpu().numpy()
    if x.dim() == 3:
        x_bits = x[:2].contiguous().view(layer.torch.int16).cpu().numpy().view(np.uint16)
    else:   # routed: the first rows of the token batch stand in for the two experts' rows
        rows = int(min(64, x.size(0) // 2))
        x_bits = x[:2 * rows].contiguous().view(layer.torch.int16).cpu().numpy().view(np.uint16).reshape(2, rows, -1)
        cnt[:2] = np.minimum(np.maximum(cnt[:2], 1), rows)
    cnt[:2] = np.minimum(cnt[:2], 64)
    t0 = time.perf_counter()
    flops, passes = 0.0, 0
    while True:
        flops += cpu_layer_pass(orc, host_sample, x_bits, cnt, g1)
        passes += 1
        if time.perf_counter() - t0 > budget_s or passes >= 3:
            break
    dt = time.perf_counter() - t0
    return dict(value=flops / dt / 1e12, unit="TFLOP/s", cores=os.cpu_count(), kind="port",
                sample=f"{passes} pass(es) over experts 0-1 of the workload, up to 64 rows each: numpy oracle quantizers + "
                       f"weight dequantisation + fp32 matmuls (BLAS threads: all cores), {dt:.1f} s")


# ------------------------------------------------------------------------------------------------
# expert-parallel headline (c4), N >= 1
# ------------------------------------------------------------------------------------------------

EP_PHASES = ("send_plan", "quant_rows", "pack_wire_rows", "all_to_all_dispatch", "dispatch_plan", "scatter_fp4_wire",
             "group_mm_gate_up", "zero_rows", "group_mm_down", "all_to_all_combine", "moe_finalize")


def run_expert_parallel(args, wl_name, wl, rank, world, local_rank, device):
    """Experts sharded over the ranks; see the module docstring for a pass.  Through torch.ops.paired_nvfp4.* and
    paired_nvfp4_kernels.ep."""
    import torch
    import torch.distributed as dist
    import paired_nvfp4_kernels
    from paired_nvfp4_kernels import _cabi, ep
    ops = torch.ops.paired_nvfp4
    H, I, T, topk = wl["hidden"], wl["inter"], wl["tokens"], wl["topk"]
    E_local = wl["E"] // world
    # per-rank tokens are fixed, so the load per expert grows with the number of ranks
    cap = max(wl["cap"], 2 * T * topk * world // wl["E"])
    slab = ep.slab_rows(T, topk, world, args.slab_headroom)
    cfg = wl["config_id"] if args.config_id is None else args.config_id
    names = _cabi.group_mm_config_names()
    cluster_m = 2 if names[cfg].split("_")[1] == "2sm" else 1
    fused_cfg = {6: 0, 7: 0, 4: 1, 5: 2, 0: 3, 1: 5, 2: 4, 3: 4, 8: 4}[cfg]
    fused_cm = 2 if _cabi.group_mm_swiglu_config_names()[fused_cfg].split("_")[1] == "2sm" else 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    copies = 1 if world == 1 else 2          # at N = 1 a pass streams 3.9 GB of weights: L2 never holds them
    first = rank * E_local
    weights = [make_expert_weights(wl, device, range(first, first + E_local), copy=c)[0] for c in range(copies)]
    seed = wl["seed"] + 100 * rank
    g = torch.Generator(device=device).manual_seed(seed)
    ids_np, w_np = topk_ids(wl, T, wl["E"], seed)
    x = torch.randn((T, H), generator=g, device=device).to(torch.bfloat16)
    ids, rw = torch.from_numpy(ids_np).to(device), torch.from_numpy(w_np).to(device)
    g1 = (6.0 * 448.0 / x.abs().max().float().clamp(min=1e-6)).reshape(1)
    if world > 1:    # one shared scale: rows are quantized before they travel
        dist.all_reduce(g1, op=dist.ReduceOp.MIN)
    al1 = (1.0 / g1).expand(E_local).contiguous()

    direct = world > 1 and args.exchange == "direct"
    peers, exchange_note = None, ""
    if direct:
        try:      # raises on every rank or on none
            peers = ep.PeerBuffers(world, rank, slab, H, int(_cabi.lib.pnv_wire_row_bytes(H)), device)
        except RuntimeError as ex:
            direct, exchange_note = False, f" ({ex}; fell back to the all-to-alls)"

    def make_ffn(w, g2, al2, peers=None):
        return ep.ExpertParallelFFN((w["a13"], w["e13"], w["s13"]), (w["a2"], w["e2"], w["s2"]), H, I, cap, al1, al2, g1, g2,
                                    slab, fused_config=fused_cfg, config_id=cfg, cluster_m=cluster_m, fused_cluster_m=fused_cm, world=world,
                                    rank=rank, peers=peers)

    # second quantizer's scales from the activation range of one unfused pass over the received rows
    ones = torch.ones(E_local, device=device)
    probe = make_ffn(weights[0], ones, ones)
    wire, _ = probe.plan_and_pack(x, ids)
    recv = probe.exchange(wire)
    counts, route_dest, src_tok, _ = ops.dispatch_plan(probe.ops.wire_expert_ids(recv), 0, E_local, cap)
    b1, sfb1 = ops.scatter_fp4_wire(recv, H, src_tok, counts, cap)
    h = torch.empty((E_local, cap, 2 * I), dtype=torch.bfloat16, device=device)
    ops.group_mm(h, weights[0]["a13"], weights[0]["e13"], weights[0]["s13"], b1, sfb1, al1, counts, 2 * I, H, cfg, cluster_m, 1)
    y = ops.gated_act(h, True)
    live = torch.arange(cap, device=device)[None, :] < counts[:, None]
    amax = torch.where(live[..., None], y.abs().float(), torch.zeros((), device=device)).amax(dim=(1, 2))
    g2 = (6.0 * 448.0 / amax.clamp(min=1e-6)).contiguous()
    al2 = (1.0 / g2).contiguous()
    del h, y, b1, sfb1, wire, recv, probe
    ffns = [make_ffn(w, g2, al2, peers) for w in weights]
    out = torch.empty((T, H), dtype=torch.bfloat16, device=device)

    def one_pass(i, mark=None):
        return ffns[i % len(ffns)].forward(x, ids, rw, out, mark)

    for i in range(3):
        _, counts, route_slot = one_pass(i)
    kept = int(counts.sum().item())
    slab_drops = int((route_slot < 0).sum().item())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(3):
        one_pass(i)
    e1.record()
    barrier()
    est = torch.tensor([e0.elapsed_time(e1) / 3 * 1e-3], device=device)
    if world > 1:
        dist.all_reduce(est, op=dist.ReduceOp.MAX)
    passes = args.passes or passes_for(float(est.item()), args.steps)
    warm = max(args.warmup, 3)
    for i in range(warm * passes):
        one_pass(i)
    step_evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    with ClockSampler(local_rank) as clocks:
        step_evs[0].record()
        for s in range(args.steps):
            for p_ in range(passes):
                one_pass(s * passes + p_)
            step_evs[s + 1].record()
        barrier()
    ms_total = torch.tensor([step_evs[0].elapsed_time(step_evs[args.steps])], device=device)
    if world > 1:
        dist.all_reduce(ms_total, op=dist.ReduceOp.MAX)
    ms_step = float(ms_total.item()) / args.steps
    step_ms = np.array([step_evs[s].elapsed_time(step_evs[s + 1]) for s in range(args.steps)])
    f = torch.tensor([2.0 * kept * (2 * I * H + H * I)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(f)
    flops_pass = float(f.item())
    pass_s = ms_step * 1e-3 / passes
    value = flops_pass / pass_s / 1e12

    # per-phase breakdown (a separate, short run: the events between launches would perturb the timed region)
    n_prof = 5
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(len(EP_PHASES) + 1)] for _ in range(n_prof)]
    barrier()
    for i in range(n_prof):
        it = iter(evs[i][1:])
        evs[i][0].record()
        one_pass(i, mark=lambda name, it=it: next(it).record())
    barrier()
    phases = {n: float(np.mean([ev[j].elapsed_time(ev[j + 1]) for ev in evs])) * 1e3 for j, n in enumerate(EP_PHASES)}
    r13, r2 = gemm_rooflines(wl_name if world == 1 and args.experts is None else None, H, I, kept, int((counts > 0).sum().item()), True,
                             phases["group_mm_gate_up"] * 1e-6, phases["group_mm_down"] * 1e-6)
    dominant = r13 if r13["launch_us"] >= r2["launch_us"] else r2

    # parity of the exchanged result: rank 0 recomputes its first tokens with the single-GPU operators
    parity = ep_parity_check(wl, device, ffns[0], x, ids, rw, g1, g2, cfg, cluster_m, fused_cfg, fused_cm, world, rank)
    if world > 1:
        dist.barrier()

    # end to end: the tokens start in pinned host memory and the layer output returns there
    e2e = None
    if not args.no_e2e:
        # as a serving loop would run it: the copy in, the layer and the copy out of consecutive passes overlap
        # (two device buffers each way, a stream for each direction beside the compute stream)
        host_x, host_out = x.cpu().pin_memory(), torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
        dev_x = [torch.empty_like(x) for _ in range(2)]
        dev_out = [torch.empty((T, H), dtype=torch.bfloat16, device=device) for _ in range(2)]
        cur, s_in, s_out = torch.cuda.current_stream(device), torch.cuda.Stream(device), torch.cuda.Stream(device)
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_back = [torch.cuda.Event() for _ in range(2)]

        def run(n):
            for i in range(n):
                k = i & 1
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(ev_done[k])        # pass i - 2 has read dev_x[k]
                    dev_x[k].copy_(host_x, non_blocking=True)
                    ev_in[k].record(s_in)
                cur.wait_event(ev_in[k])
                if i >= 2:
                    cur.wait_event(ev_back[k])             # pass i - 2's output has left dev_out[k]
                ffns[i % len(ffns)].forward(dev_x[k], ids, rw, dev_out[k])
                ev_done[k].record(cur)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[k])
                    host_out.copy_(dev_out[k], non_blocking=True)
                    ev_back[k].record(s_out)
            cur.wait_stream(s_out)

        run(4)
        torch.cuda.synchronize()
        want = ffns[3 % len(ffns)].forward(x, ids, rw)[0]          # the last of the four passes, device resident
        torch.cuda.synchronize()
        assert torch.equal(host_out.to(device), want), "the pipelined passes do not reproduce the device-resident pass"
        del want
        n = max(6, min(args.steps * passes, 50))
        barrier()
        e0.record()
        run(n)
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item()) / n
        e2e = dict(value=flops_pass / (ms_e2e * 1e-3) / 1e12, unit="TFLOP/s", ms_per_pass=ms_e2e,
                   h2d_bytes_per_step=host_x.numel() * 2 * world * passes, d2h_bytes_per_step=host_out.numel() * 2 * world * passes,
                   passes=n, mode="eager operator calls; the host->device copy, the layer and the device->host copy of "
                                   "consecutive passes overlap (two device buffers each way, one stream per direction)")
    if peers is not None:
        peers.close()          # a collective: before the other ranks leave
    if rank != 0:
        return None
    rb = _cabi.lib.pnv_wire_row_bytes(H)
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "e2m1 x e2m1 -> f32", "data": "synthetic",
        "config": {"workload": f"{wl_name}: {wl['desc']}", "experts": wl["E"], "experts_per_gpu": E_local,
                   "hidden": H, "intermediate": I, "cap": cap, "tokens_per_gpu": T, "topk": topk,
                   "routed_rows_kept_rank0": kept, "slab_rows": slab, "routings_dropped_by_slab_rank0": slab_drops,
                   "tile_config": names[cfg], "fused_swiglu_epilogue": True, "parallelism": f"ep{world}",
                   "passes_per_step": passes,
                   "exchange": ("direct: pack_wire_rows stores NVFP4 wire rows into the receivers' buffers and the down "
                                "GEMM's epilogue stores bf16 expert outputs into the senders' buffers over NVLink (peer memory, "
                                "plain stores); two one-element all-reduces per pass order them; the phases named all_to_all_* "
                                "are those fences" if direct else
                                "one equal-split NCCL all_to_all_single each way: NVFP4 wire rows out, bf16 rows back; "
                                "routing planned on the device inside every pass" + exchange_note) if world > 1 else
                               "N = 1: both all-to-alls are the identity, everything else is the N > 1 pass",
                   "l2": "inputs larger than L2" + ("; two weight copies alternate" if copies > 1 else "")},
        "layer_us": pass_s * 1e6, "step_ms_mean": float(step_ms.mean()), "step_ms_p10": float(np.percentile(step_ms, 10)),
        "phases_us": phases,
        "nvlink_bytes_per_gpu_per_pass": (world - 1) * slab * (rb + 2 * H) if world > 1 else 0,
        "roofline": dominant, "rooflines": {"group_mm_gate_up": r13, "group_mm_down": r2},
        "ep_parity": parity, "cpu_baseline": None, "e2e": e2e,
        # our kernels per pass: 2 x dispatch_plan (3 launches each), quant_rows, pack_wire_rows, scatter_fp4_wire, 2 x group_mm,
        # zero_rows, moe_finalize (the all-to-alls are NCCL's)
        "gpu_launches": 13 * passes * args.steps,
        "clocks": clocks.summary(),
    }
    return line


def ep_parity_check(wl, device, ffn, x, ids, rw, g1, g2_local, cfg, cluster_m, fused_cfg, fused_cm, world, rank, n_tok=64):
    """Rank 0 recomputes the first n_tok tokens of its batch on its own GPU through the single-GPU operators (the
    experts they route to regenerate from the seed; their second-quantizer scales are gathered from their
    owners) and compares with the exchanged result, bit for bit.  Every rank takes part in the extra pass."""
    import torch
    import torch.distributed as dist
    out, _, route_slot = ffn.forward(x, ids, rw)          # weight copy 0
    torch.cuda.synchronize()
    if world > 1:
        g2_all = [torch.empty_like(g2_local) for _ in range(world)]
        dist.all_gather(g2_all, g2_local)
        g2_all = torch.cat(g2_all)
    else:
        g2_all = g2_local
    if rank != 0:
        return None
    return _ep_parity_rank0(wl, device, out, route_slot, x, ids, rw, g1, g2_all, cfg, cluster_m, fused_cfg, fused_cm, n_tok)


def _ep_parity_rank0(wl, device, out, route_slot, x, ids, rw, g1, g2_all, cfg, cluster_m, fused_cfg, fused_cm, n_tok):
    import torch
    ops = torch.ops.paired_nvfp4
    H, I = wl["hidden"], wl["inter"]
    sub_ids = ids[:n_tok]
    needed = torch.unique(sub_ids).cpu().numpy()
    remap = torch.full((wl["E"],), -1, dtype=torch.int64, device=device)
    remap[torch.from_numpy(needed).to(device)] = torch.arange(len(needed), device=device)
    w, _ = make_expert_weights(wl, device, needed, copy=0)
    n = len(needed)
    local_ids = remap[sub_ids]
    # routings the slab dropped stay dropped
    local_ids = torch.where(route_slot[:n_tok] < 0, torch.full_like(local_ids, -1), local_ids)
    ccap = 128
    counts, route_dest, src_tok, _ = ops.dispatch_plan(local_ids, 0, n, ccap)
    q, q_sf = ops.quant_rows(x[:n_tok].contiguous(), g1)
    b1, sfb1 = ops.scatter_fp4_planned(q, q_sf, src_tok, counts, ccap)
    sel = torch.from_numpy(needed).to(device)
    g2 = g2_all[sel].contiguous()
    al1 = (1.0 / g1).expand(n).contiguous()
    b2, sfb2 = ops.group_mm_swiglu_quant(w["a13"], w["e13"], w["s13"], b1, sfb1, al1, counts, g2, 2 * I, H, fused_cfg,
                                         fused_cm, 1)
    y = torch.empty((n, ccap, H), dtype=torch.bfloat16, device=device)
    ops.group_mm(y, w["a2"], w["e2"], w["s2"], b2, sfb2, (1.0 / g2).contiguous(), counts, H, I, cfg, cluster_m, 1)
    want = torch.empty((n_tok, H), dtype=torch.bfloat16, device=device)
    ops.moe_finalize(want, y, route_dest, rw[:n_tok].contiguous())
    torch.cuda.synchronize()
    got = out[:n_tok]
    a, b = got.float(), want.float()
    rel = float((a - b).norm() / b.norm().clamp(min=1e-30))
    return {"tokens": n_tok, "experts_recomputed": int(n), "bit_exact": bool(torch.equal(got, want)), "rel_frobenius": rel}


# ------------------------------------------------------------------------------------------------

def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl_name = args.workload or "c4"
    wl = WORKLOADS[wl_name]
    if args.experts is not None:
        assert wl["routing"] in ("topk", "zipf") and 0 < args.experts <= wl["E"], "--experts: a routed workload, at most its own count"
        wl = dict(wl, E=args.experts, tokens=max(1, wl["tokens"] * args.experts // wl["E"]),
                  desc=f"{wl['desc']} (cut to {args.experts} experts for a profiler capture)")

    if args.impl == "reference":
        return run_reference_arm(args, wl_name, wl, rank)

    import torch
    import paired_nvfp4_kernels  # noqa: F401  (loads the CUDA library; raises if it is missing)
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
        assert wl_name == "c4", "N > 1 runs the expert-parallel workload (c4)"
    assert wl["E"] % world == 0

    if wl_name == "c4":
        line = run_expert_parallel(args, wl_name, wl, rank, world, local_rank, device)
        if rank == 0 and world == 1:
            subs = {}
            if not args.no_sub_workloads:
                for name in ("c2", "c3"):
                    sub = run_local_workload(name, WORKLOADS[name], device, args, steps=max(5, min(args.steps, 20)),
                                             warmup=3, with_e2e=(name == "c2"), with_cpu=False)
                    sub.pop("flops_per_pass", None)
                    subs[name] = sub
            line["workloads"] = subs
            if not args.no_cpu_baseline:
                line["cpu_baseline"] = run_cpu_sample(wl)
        if rank == 0:
            print(json.dumps(line))
        if world > 1:
            torch.distributed.destroy_process_group()
        return

    with_clocks = ClockSampler(local_rank)
    res = run_local_workload(wl_name, wl, device, args, args.steps, max(args.warmup, 3), sample_clocks=with_clocks)
    line = {"metric": METRIC, "value": res.pop("value"), "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": res.pop("ms_per_step"), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "e2m1 x e2m1 -> f32", "data": "synthetic"}
    res.pop("flops_per_pass", None)
    line.update(res)
    line.setdefault("cpu_baseline", None)
    line.setdefault("e2e", None)
    line["clocks"] = with_clocks.summary()
    print(json.dumps(line))


def run_cpu_sample(wl, budget_s=12.0):
    """CPU baseline of the headline workload: one expert's weights through the reference's reference.py (prune +
    quantize, when oracle/_ref holds it), then 64 routed rows through the numpy oracle (quantizers, weight
    dequantisation, fp32 matmuls), a slice of the output features; dense-equivalent TFLOP/s of the matmuls over
    the whole sample time."""
    from oracle import paired_nvfp4_oracle as orc
    ref = load_reference_py()
    H, I = wl["hidden"], wl["inter"]
    rows, m13, m2 = 64, min(2 * I, 1024), min(H, 512)
    t0 = time.perf_counter()
    p13, s13 = cpu_weight_half(ref, orc, m13, H, wl["wstd"], wl["seed"])
    p2, s2 = cpu_weight_half(ref, orc, m2, I, wl["wstd"], wl["seed"] + 1)
    t_w = time.perf_counter() - t0
    rng = np.random.default_rng(wl["seed"])
    x = orc.f32_to_bf16_bits(rng.standard_normal((1, rows, H)).astype(np.float32))
    x2 = orc.f32_to_bf16_bits(rng.standard_normal((1, rows, 2 * I)).astype(np.float32))
    cnt, one = np.array([rows], np.int32), np.ones(1, np.float32)
    flops, passes = 0.0, 0
    t1 = time.perf_counter()
    while True:
        b1, _, sfb1 = orc.quant_act(x, one, cnt)
        orc.group_mm(orc.dequantize_weight(p13, s13), b1, sfb1, one, cnt)
        b2, _, sfb2, _ = orc.silu_mul_quant_act(x2, one, cnt)
        orc.group_mm(orc.dequantize_weight(p2, s2), b2, sfb2, one, cnt)
        flops += 2.0 * rows * (m13 * H + m2 * I)
        passes += 1
        if time.perf_counter() - t1 > budget_s or passes >= 400:
            break
    dt = time.perf_counter() - t1
    return dict(value=flops / dt / 1e12, unit="TFLOP/s", cores=os.cpu_count(), kind="_ref+port" if ref is not None else "port",
                sample=f"weights of {m13} gate_up and {m2} down features pruned + quantized by "
                       f"{'the reference reference.py' if ref is not None else 'the numpy port'} ({t_w:.1f} s, not in the rate); "
                       f"{passes} pass(es) of {rows} routed rows: numpy oracle quantizers + weight dequantisation + fp32 "
                       f"matmuls (BLAS threads: all cores), {dt:.1f} s")


def run_reference_arm(args, wl_name, wl, rank):
    """The reference's CPU implementation of the path on the host cores: the weight spec from the reference's own
    reference.py (oracle/_ref, when present), the quantizers and the fp32 dequantised matmul restated in numpy by
    the oracle; each step is a bounded sample of the workload."""
    if rank != 0:
        return
    from oracle import paired_nvfp4_oracle as orc
    ref = load_reference_py()
    H, I = wl["hidden"], wl["inter"]
    rows = 16 if wl["routing"] in ("counts", "one") else 64
    m13, m2 = min(2 * I, 1024), min(H, 512)   # a slice of output features of one expert per step
    p13, s13 = cpu_weight_half(ref, orc, m13, H, wl["wstd"], wl["seed"])
    p2, s2 = cpu_weight_half(ref, orc, m2, I, wl["wstd"], wl["seed"] + 1)
    rng = np.random.default_rng(wl["seed"])
    x = orc.f32_to_bf16_bits(rng.standard_normal((1, rows, H)).astype(np.float32))
    x2 = orc.f32_to_bf16_bits(rng.standard_normal((1, rows, 2 * I)).astype(np.float32))
    cnt = np.array([rows], np.int32)
    one = np.ones(1, np.float32)
    flops_step = 2.0 * rows * (m13 * H + m2 * I)
    dq = (lambda p, s: ref.dequantize_weight(_t(p), _t(s).view(_f8())).numpy()) if ref is not None else orc.dequantize_weight

    def step():
        b1, _, sfb1 = orc.quant_act(x, one, cnt)
        orc.group_mm(dq(p13, s13), b1, sfb1, one, cnt)
        b2, _, sfb2, _ = orc.silu_mul_quant_act(x2, one, cnt)
        orc.group_mm(dq(p2, s2), b2, sfb2, one, cnt)

    warm = min(max(args.warmup, 0), 10)
    for _ in range(warm):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    ms = dt / args.steps * 1e3
    value = flops_step / (ms * 1e-3) / 1e12
    kind = "_ref+port" if ref is not None else "port"
    sample = (f"per step: one expert, {rows} rows, {m13} of {2 * I} gate_up features and {m2} of {H} down features: "
              f"weight dequantisation by {'the reference reference.py' if ref is not None else 'the numpy port'}, numpy "
              "oracle quantizers + fp32 matmuls")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{wl_name}: {wl['desc']}", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a))


def _f8():
    import torch
    return torch.float8_e4m3fn


if __name__ == "__main__":
    main()
