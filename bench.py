#!/usr/bin/env python
"""Benchmark of the paired-4:8 sparse NVFP4 grouped MoE GEMM path on B200.

    python bench.py --gpus 1 --steps K --warmup W [--workload c2|c3|c4|c5] [--impl reference]

One "step" is one expert-FFN pass of a MoE layer over one batch of synthetic, seeded, model-shaped
input: activation quantizer -> group_mm (gate_up) -> gated activation + quantizer -> group_mm (down).
The default single-GPU workload is the decode configuration (Mixtral-8x7B-shaped, memory bound).
`value` is dense-equivalent TFLOP/s of the two grouped GEMMs over the whole step with every input
resident in HBM; `e2e` is the same metric through torch.ops.paired_nvfp4.* with the activations in
pinned host memory (copy in, layer, copy out, inside the timed region).  The line also carries the
roofline of the dominant kernel and a CPU baseline (the numpy oracle on the host cores).

`--impl reference` times that CPU implementation alone, on bounded samples of the same workload.
"""
import argparse
import ctypes
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

FALLBACK_HBM_GBS = 6650.0   # earlier measurement on this pool, used only without MEASURED_PEAKS.json

# dram__bytes_read.sum + dram__bytes_write.sum of one gate_up group_mm launch, from the ncu captures
# summarised under profiles/ (same workload, so no scaling)
NCU_TRAFFIC_BYTES = {"c2": 328.10e6, "c3": 337.87e6}

# name -> dict(E, hidden, inter, max_n/cap, routing)
WORKLOADS = {
    # Mixtral-8x7B expert FFN, decode: per-expert counts uniform in [1, 16]
    "c2": dict(desc="decode Mixtral-8x7B-shaped expert FFN", E=8, hidden=4096, inter=14336, cap=16,
               routing="counts", seed=1001, config_id=7, wstd=0.02),
    # Qwen3-30B-A3B MoE, prefill: 16384 tokens, top-8 of 128, cap 2048
    "c3": dict(desc="prefill Qwen3-30B-A3B-shaped MoE", E=128, hidden=2048, inter=768, cap=2048,
               routing="topk", tokens=16384, topk=8, seed=1002, config_id=8, wstd=0.02),
    # DeepSeek-V3 MoE, one expert-parallel rank's share: 8192 tokens, top-8 of 256
    "c4": dict(desc="DeepSeek-V3-shaped MoE, expert parallel", E=256, hidden=7168, inter=2048, cap=1024,
               routing="topk", tokens=8192, topk=8, seed=1003, config_id=8, wstd=0.02),
    # the per-rank shape of c4 at 8 ranks (32 local experts, 65536 routed rows), without the exchange
    "c4r8": dict(desc="DeepSeek-V3-shaped MoE, one rank's expert shard at 8 ranks", E=32, hidden=7168, inter=2048,
                 cap=4096, routing="topk", tokens=8192, topk=8, seed=1005, config_id=8, wstd=0.02),
    # skewed routing: Zipf(1.2) expert popularity, top-4 of 128 over 8192 tokens, cap 4096
    "c5": dict(desc="skewed-routing MoE (Zipf 1.2)", E=128, hidden=3072, inter=3072, cap=4096,
               routing="zipf", tokens=8192, topk=4, seed=1004, config_id=8, wstd=0.02),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--config-id", type=int, default=None, help="group_mm tile variant override")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--unfused", action="store_true", help="separate silu_mul_quant_act launch instead of the fused GEMM1 epilogue")
    ap.add_argument("--ep-sm-margin", type=int, default=0, help="N > 1: SMs left free for the collectives while slices overlap")
    ap.add_argument("--ep-chunks", type=int, default=1, help="N > 1: token slices whose exchanges overlap the GEMMs (1 = no overlap)")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------
# byte / flop accounting (algorithmic: what the math needs, independent of the implementation)
# ------------------------------------------------------------------------------------------------

def _ru(a, b):
    return -(-a // b) * b


def gemm_bytes(active, M, K, rows):
    """Weights of the active experts (codes + metadata + scales) + activation codes/scales in +
    bf16 out; the same formula the reference's tools/bench_moe.py uses (sparse_bytes)."""
    kb = -(-K // 32)
    w = active * (M * K // 4 + _ru(M, 128) * _ru(K, 256) // 16 + _ru(M, 128) * _ru(kb, 4))
    return w + rows * (K // 2 + K // 32) + rows * 2 * M


def layer_accounting(wl, counts, fused=True):
    rows = int(counts.sum())
    active = int((counts > 0).sum())
    H, I = wl["hidden"], wl["inter"]
    flops = 2.0 * rows * (2 * I * H + H * I)
    b13 = gemm_bytes(active, 2 * I, H, rows)
    b2 = gemm_bytes(active, H, I, rows)
    quant1 = rows * (2 * H + H // 2 + H // 32)
    quant2 = rows * (4 * I + I // 2 + I // 32)
    if fused:   # GEMM1 writes GEMM2's codes + scales instead of bf16; no separate activation pass
        b13 += rows * (I // 2 + I // 32) - rows * 2 * (2 * I)
        quant2 = 0
    return dict(rows=rows, active=active, flops=flops, bytes_w13=b13, bytes_w2=b2,
                bytes_total=b13 + b2 + quant1 + quant2)


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


def plan_from_ids(ids, first_expert, num_local, cap):
    """Token-major flat plan with stable per-expert ranks (drop = num_local * cap)."""
    T, topk = ids.shape
    flat = ids.reshape(-1) - first_expert
    n = flat.size
    local = (flat >= 0) & (flat < num_local)
    key = np.where(local, flat, num_local)
    order = np.argsort(key, kind="stable")
    sorted_e = key[order]
    starts = np.searchsorted(sorted_e, np.arange(num_local + 1))
    rank = np.empty(n, dtype=np.int64)
    rank[order] = np.arange(n) - starts[np.minimum(sorted_e, num_local)]
    dest = np.full(n, num_local * cap, dtype=np.int64)
    ok = local & (rank < cap)
    dest[ok] = flat[ok] * cap + rank[ok]
    counts = np.minimum(starts[1:] - starts[:-1], cap)[:num_local].astype(np.int32)
    return (np.arange(n, dtype=np.int64) // topk), dest, counts


class Layer:
    """Device state of one expert-FFN layer and the four launches of a step, through the C ABI."""

    def __init__(self, wl, device, config_id=None, copies=2, E_local=None, first_expert=0, seed_shift=0, fused=True):
        import torch
        from paired_nvfp4_kernels import _cabi, reference as wref
        self.torch, self.lib, self.cabi = torch, _cabi.lib, _cabi
        self.wl, self.dev = wl, device
        self.E = E_local if E_local is not None else wl["E"]
        self.H, self.I, self.cap = wl["hidden"], wl["inter"], wl["cap"]
        self.cfg = wl["config_id"] if config_id is None else config_id
        self.fused = fused
        names = _cabi.group_mm_config_names()
        self.cluster_m = 2 if names[self.cfg].split("_")[1] == "2sm" else 1
        # fused variant with the same tile as the chosen group_mm variant
        fmap = {6: 0, 7: 0, 4: 1, 5: 2, 0: 3, 1: 3, 2: 4, 3: 4, 8: 4}
        self.fused_cfg = fmap.get(self.cfg, 3)
        if fused:
            self.cluster_m = 2 if _cabi.group_mm_swiglu_config_names()[self.fused_cfg].split("_")[1] == "2sm" else self.cluster_m
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        ops = torch.ops.paired_nvfp4
        E, H, I = self.E, self.H, self.I
        # weights: N(0, wstd), pruned paired-4:8, NVFP4; generated per expert on the GPU with the
        # package's torch weight spec (bit-identical to the reference's reference.py), then compressed
        self.weights = []
        self.host_sample = {}
        for c in range(copies):
            parts13, parts2 = [], []
            for e in range(E):
                g = torch.Generator(device=device).manual_seed(wl["seed"] * 7919 + 1000 * c + first_expert + e + seed_shift)
                w13 = torch.randn((1, 2 * I, H), generator=g, device=device) * wl["wstd"]
                w2 = torch.randn((1, H, I), generator=g, device=device) * wl["wstd"]
                p13, s13, _ = wref.quantize_weight(wref.prune_paired_4of8(w13))
                if fused:   # gate/up rows interleaved in 64-row blocks for the fused epilogue
                    import paired_nvfp4_kernels as pnk
                    perm = pnk.interleave_gate_up_rows(I, device=device)
                    p13, s13 = p13[:, perm].contiguous(), s13[:, perm].contiguous()
                p2, s2, _ = wref.quantize_weight(wref.prune_paired_4of8(w2))
                if c == 0 and e < 2:
                    self.host_sample[e] = tuple(t.cpu().numpy() for t in (p13, s13, p2, s2))
                parts13.append(ops.compress(p13, s13, H))
                parts2.append(ops.compress(p2, s2, I))
                del w13, w2, p13, s13, p2, s2
            cat = lambda parts, i: torch.cat([p[i] for p in parts], 0) if i < 2 else torch.cat([p[i] for p in parts])
            self.weights.append(dict(a13=cat(parts13, 0), e13=cat(parts13, 1), s13=cat(parts13, 2),
                                     a2=cat(parts2, 0), e2=cat(parts2, 1), s2=cat(parts2, 2)))
            del parts13, parts2
        u8 = dict(dtype=torch.uint8, device=device)
        self.b1 = torch.empty((E * self.cap + 1, H // 2), **u8)
        self.sfb1 = torch.empty((_cabi.sf_numel(self.cap, H, E),), **u8)
        self.out1 = torch.zeros((E, self.cap, 2 * I), dtype=torch.bfloat16, device=device)
        self.b2 = torch.empty((E, self.cap, I // 2), **u8)
        self.sfb2 = torch.empty((_cabi.sf_numel(self.cap, I, E),), **u8)
        self.out2 = torch.zeros((E, self.cap, H), dtype=torch.bfloat16, device=device)
        self.ev = None

    def set_inputs(self, x, counts, g1, a1, g2, a2, flat_tok=None, dest=None, topk_w=None):
        """x: bf16 [E, cap, H] (decode) or [T, H] (routed).  All device tensors."""
        self.x, self.counts, self.g1, self.al1, self.g2, self.al2 = x, counts, g1, a1, g2, a2
        self.flat_tok, self.dest, self.topk_w = flat_tok, dest, topk_w

    def step(self, stream, c=0, events=None):
        lib, ck = self.lib, self.cabi.check
        w = self.weights[c % len(self.weights)]
        E, H, I, cap, sm = self.E, self.H, self.I, self.cap, self.sm_count
        if self.flat_tok is None:
            ck(lib.pnv_quant_act(self.x.data_ptr(), self.g1.data_ptr(), 1, self.counts.data_ptr(), E, cap, H,
                                 self.b1.data_ptr(), self.sfb1.data_ptr(), sm, stream))
        else:
            ck(lib.pnv_scatter_quant_act(self.x.data_ptr(), self.flat_tok.data_ptr(), self.dest.data_ptr(),
                                         self.topk_w.data_ptr() if self.topk_w is not None else None,
                                         self.g1.data_ptr(), 1, self.flat_tok.numel(), H, E, cap,
                                         self.b1.data_ptr(), self.sfb1.data_ptr(), sm, stream))
        if events:
            events[0].record()
        if self.fused:
            ck(lib.pnv_group_mm_swiglu_quant(self.b2.data_ptr(), self.sfb2.data_ptr(), w["a13"].data_ptr(),
                                             w["e13"].data_ptr(), w["s13"].data_ptr(), self.b1.data_ptr(),
                                             self.sfb1.data_ptr(), self.al1.data_ptr(), self.counts.data_ptr(),
                                             self.g2.data_ptr(), 1, E, 2 * I, H, cap, self.fused_cfg, self.cluster_m, 1,
                                             0, 1.0, -1.0, sm, 1, stream))
            if events:
                events[1].record()
                events[2].record()
        else:
            ck(lib.pnv_group_mm(self.out1.data_ptr(), w["a13"].data_ptr(), w["e13"].data_ptr(), w["s13"].data_ptr(),
                                self.b1.data_ptr(), self.sfb1.data_ptr(), self.al1.data_ptr(), self.counts.data_ptr(),
                                E, 2 * I, H, cap, self.cfg, self.cluster_m, 1, sm, 1, stream))
            if events:
                events[1].record()
            ck(lib.pnv_silu_mul_quant_act(self.out1.data_ptr(), self.g2.data_ptr(), 1, self.counts.data_ptr(), E, cap,
                                          I, 0, 0, 1.0, -1.0, self.b2.data_ptr(), self.sfb2.data_ptr(), sm, stream))
            if events:
                events[2].record()
        ck(lib.pnv_group_mm(self.out2.data_ptr(), w["a2"].data_ptr(), w["e2"].data_ptr(), w["s2"].data_ptr(),
                            self.b2.data_ptr(), self.sfb2.data_ptr(), self.al2.data_ptr(), self.counts.data_ptr(),
                            E, H, I, cap, self.cfg, self.cluster_m, 1, sm, 1, stream))
        if events:
            events[3].record()


def make_activation_inputs(wl, layer, rank, world, device):
    """Seeded activations / routing for this rank; returns kwargs for Layer.set_inputs and counts."""
    import torch
    E, H, cap = layer.E, layer.H, layer.cap
    seed = wl["seed"] + 100 * rank
    g = torch.Generator(device=device).manual_seed(seed)
    if wl["routing"] == "counts":
        counts = np.random.default_rng(seed).integers(1, cap + 1, E).astype(np.int32)
        x = torch.randn((E, cap, H), generator=g, device=device).to(torch.bfloat16)
        flat_tok = dest = topk_w = None
        amax = torch.stack([x[e, :int(counts[e])].abs().max() for e in range(E)]).float()
    else:
        T = wl["tokens"]
        ids, w = topk_ids(wl, T, wl["E"], seed)
        first = rank * E if world > 1 else 0
        ft, d, counts = plan_from_ids(ids, first, E, cap)
        x = torch.randn((T, H), generator=g, device=device).to(torch.bfloat16)
        flat_tok = torch.from_numpy(ft).to(device)
        dest = torch.from_numpy(d).to(device)
        topk_w = None   # router weights are applied at combine time
        amax = x.abs().max().float().expand(E).contiguous()
        layer.global_ids = torch.from_numpy(ids).to(device)
        layer.router_w = torch.from_numpy(w).to(device)
    g1 = (6.0 * 448.0 / amax.clamp(min=1e-6)).contiguous()
    return dict(x=x, counts=torch.from_numpy(counts).to(device), g1=g1, a1=(1.0 / g1).contiguous(),
                flat_tok=flat_tok, dest=dest, topk_w=topk_w), counts


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
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": []}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# ------------------------------------------------------------------------------------------------
# CPU baseline: the numpy oracle (a port of the reference's reference.py + quantizer restatements)
# ------------------------------------------------------------------------------------------------

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


def run_cpu_baseline(layer, inputs, counts, budget_s=15.0):
    from oracle import paired_nvfp4_oracle as orc
    x = inputs["x"]
    if x.dim() != 3:
        return None
    x_bits = x[:2].contiguous().view(layer.torch.int16).cpu().numpy().view(np.uint16)
    g1 = inputs["g1"].cpu().numpy()
    t0 = time.perf_counter()
    flops, passes = 0.0, 0
    while True:
        flops += cpu_layer_pass(orc, layer.host_sample, x_bits, counts, g1)
        passes += 1
        if time.perf_counter() - t0 > budget_s or passes >= 3:
            break
    dt = time.perf_counter() - t0
    return dict(value=flops / dt / 1e12, unit="TFLOP/s", cores=os.cpu_count(), kind="port",
                sample=f"{passes} pass(es) over experts 0-1 of the workload, every row: numpy oracle quantizers + "
                       f"weight dequantisation + fp32 matmuls (BLAS threads: all cores), {dt:.1f} s")


# ------------------------------------------------------------------------------------------------

def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl_name = args.workload or ("c2" if args.gpus == 1 else "c4")
    wl = WORKLOADS[wl_name]

    if args.impl == "reference":
        return run_reference_arm(args, wl_name, wl, rank)

    import torch
    import paired_nvfp4_kernels  # noqa: F401  (loads the CUDA library; raises if it is missing)
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    assert wl["E"] % world == 0
    E_local = wl["E"] // world
    if world > 1:
        assert wl["routing"] != "counts", "expert parallelism needs a routed workload (c3, c4, c5)"
        assert not args.unfused, "the expert-parallel step always uses the fused gate_up epilogue"
        # per-rank tokens are fixed, so the load per expert grows with the number of ranks
        wl = dict(wl, cap=max(wl["cap"], 2 * wl["tokens"] * wl["topk"] * world // wl["E"]))
    layer = Layer(wl, device, config_id=args.config_id, E_local=E_local, first_expert=rank * E_local,
                  fused=not args.unfused)
    inputs, counts = make_activation_inputs(wl, layer, rank, world, device)
    stream = torch.cuda.current_stream().cuda_stream
    calibrate_second_scale(layer, inputs, stream)
    acct = layer_accounting(wl, counts, fused=not args.unfused)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    if world > 1:
        return run_expert_parallel(args, wl_name, wl, layer, inputs, rank, world, local_rank, device, barrier)

    # ---- device-resident timing ---------------------------------------------------------------
    for i in range(max(args.warmup, 3)):
        layer.step(stream, c=i)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local_rank) as clocks:
        e0.record()
        for i in range(args.steps):
            layer.step(stream, c=i, events=evs[i])
        e1.record()
        barrier()
    ms_total = e0.elapsed_time(e1)
    k13 = float(np.mean([e[0].elapsed_time(e[1]) for e in evs])) * 1e-3
    kq2 = float(np.mean([e[1].elapsed_time(e[2]) for e in evs])) * 1e-3
    k2 = float(np.mean([e[2].elapsed_time(e[3]) for e in evs])) * 1e-3
    if world > 1:
        t = torch.tensor([ms_total], device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms_total = float(t.item())
        f = torch.tensor([acct["flops"]], device=device, dtype=torch.float64)
        torch.distributed.all_reduce(f)
        total_flops = float(f.item())
    else:
        total_flops = acct["flops"]
    ms_step = ms_total / args.steps
    value = total_flops / (ms_step * 1e-3) / 1e12

    # ---- end to end through the public operators, activations in pinned host memory ----------
    e2e = None
    if not args.no_e2e and world == 1:
        e2e = run_e2e(layer, inputs, wl, args, total_flops)

    # ---- roofline of the dominant kernel (the gate_up group_mm) -------------------------------
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, src = FALLBACK_HBM_GBS, "fallback"
    achieved = acct["bytes_w13"] / k13 / 1e9
    roofline = dict(bound="hbm", kernel="group_mm gate_up", achieved=achieved, peak=peak, unit="GB/s",
                    frac=achieved / peak, peak_source=src, traffic=NCU_TRAFFIC_BYTES.get(wl_name),
                    algorithmic_bytes=acct["bytes_w13"], launch_us=k13 * 1e6)

    if rank == 0:
        cpu = None
        if not args.no_cpu_baseline and world == 1:
            cpu = run_cpu_baseline(layer, inputs, counts)
        line = {
            "metric": "moe_expert_ffn_group_mm_dense_equiv_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "e2m1 x e2m1 -> f32",
            "data": "synthetic",
            "config": {"workload": f"{wl_name}: {wl['desc']}", "experts": wl["E"], "experts_per_gpu": E_local,
                       "hidden": wl["hidden"], "intermediate": wl["inter"], "cap": wl["cap"],
                       "routed_rows_rank0": acct["rows"], "tile_config": paired_nvfp4_kernels.group_mm_configs()[layer.cfg],
                       "fused_swiglu_epilogue": layer.fused,
                       "l2": "two weight copies alternate; each step streams > 3x the 126 MB L2" if wl_name == "c2"
                             else "inputs larger than L2; two weight copies alternate"},
            "layer_us": ms_step * 1e3, "hbm_gbs_layer": acct["bytes_total"] / (ms_step * 1e-3) / 1e9,
            "kernels_us": {"group_mm_gate_up": k13 * 1e6, "silu_mul_quant_act": kq2 * 1e6, "group_mm_down": k2 * 1e6},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": (3 if layer.fused else 4) * args.steps,
            "clocks": clocks.summary(),
        }
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


def run_expert_parallel(args, wl_name, wl, layer, inputs, rank, world, local_rank, device, barrier):
    """N > 1: experts sharded over the ranks; every step is dispatch (NVFP4 rows over NCCL all-to-all) ->
    dispatch_plan -> scatter -> fused gate_up group_mm -> down group_mm -> combine (all-to-all) ->
    moe_finalize, through torch.ops.paired_nvfp4.* and paired_nvfp4_kernels.ep."""
    import torch
    import torch.distributed as dist
    import paired_nvfp4_kernels
    from paired_nvfp4_kernels import ep
    H, I = layer.H, layer.I
    plan = ep.build_plan(layer.global_ids, layer.E)
    chunks = max(1, args.ep_chunks)
    if chunks > 1 and args.ep_sm_margin:
        from paired_nvfp4_kernels import ops as pyops
        pyops.set_sm_margin(args.ep_sm_margin)
    plans = ep.build_chunk_plans(layer.global_ids, layer.E, chunks) if chunks > 1 else None
    comm = torch.cuda.Stream(device=device)

    def forward(ffn, xin):
        if plans is None:
            return ffn.forward(xin, plan, rw, out)[1]
        return torch.stack(ep.forward_chunked(ffn, xin, plans, rw, out, comm)).sum(0)
    g1 = inputs["g1"][:1].contiguous()                       # one shared scale: rows are quantized before they travel
    al1 = (1.0 / g1).expand(layer.E).contiguous()
    ffns = []
    for w in layer.weights:
        ffns.append(ep.ExpertParallelFFN((w["a13"], w["e13"], w["s13"]), (w["a2"], w["e2"], w["s2"]), H, I, layer.cap,
                                         al1, layer.al2, g1, layer.g2, fused_config=layer.fused_cfg,
                                         config_id=layer.cfg, cluster_m=layer.cluster_m))
    x, rw = inputs["x"], layer.router_w
    out = torch.empty((plan.tokens, H), dtype=torch.bfloat16, device=device)
    counts = None
    for i in range(max(args.warmup, 3)):
        counts = forward(ffns[i % len(ffns)], x)
    kept = int(counts.sum().item())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local_rank) as clocks:
        e0.record()
        for i in range(args.steps):
            forward(ffns[i % len(ffns)], x)
        e1.record()
        barrier()
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    f = torch.tensor([2.0 * kept * (2 * I * H + H * I)], device=device, dtype=torch.float64)
    dist.all_reduce(f)
    total_flops = float(f.item())
    value = total_flops / (ms_step * 1e-3) / 1e12

    # end to end: the tokens start in pinned host memory and the layer output returns there
    host_x, host_out = x.cpu().pin_memory(), torch.empty((plan.tokens, H), dtype=torch.bfloat16).pin_memory()
    dev_x = torch.empty_like(x)

    def one(i):
        dev_x.copy_(host_x, non_blocking=True)
        forward(ffns[i % len(ffns)], dev_x)
        host_out.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
    for i in range(3):
        one(i)
    n = max(5, min(args.steps, 50))
    barrier()
    e0.record()
    for i in range(n):
        one(i)
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_e2e = float(t.item()) / n
    if rank == 0:
        wire = plan.n_send * (H // 2 + H // 32 + 4) + plan.n_recv * 2 * H
        print(json.dumps({
            "metric": "moe_expert_ffn_group_mm_dense_equiv_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "e2m1 x e2m1 -> f32",
            "data": "synthetic",
            "config": {"workload": f"{wl_name}: {wl['desc']}", "experts": wl["E"], "experts_per_gpu": layer.E,
                       "hidden": H, "intermediate": I, "cap": layer.cap, "tokens_per_gpu": plan.tokens,
                       "topk": plan.topk, "routed_rows_kept_rank0": kept,
                       "tile_config": paired_nvfp4_kernels.group_mm_configs()[layer.cfg],
                       "fused_swiglu_epilogue": True, "parallelism": f"ep{world}", "token_slices": chunks,
                       "exchange": "NCCL all_to_all_single: NVFP4 rows + scales + expert ids out, bf16 rows back",
                       "l2": "inputs larger than L2; two weight copies alternate"},
            "layer_us": ms_step * 1e3, "nvlink_bytes_per_gpu_per_step": wire,
            "roofline": {"bound": "tensor", "kernel": "whole expert-parallel step", "achieved": value / world,
                         "peak": 18000.0, "unit": "TFLOP/s", "frac": value / world / 18000.0,
                         "peak_source": "nominal 2:4-sparse FP4 per GPU in dense-equivalent flops (no measured FP4 peak on this pool)",
                         "traffic": None},
            "cpu_baseline": None,
            "e2e": dict(value=total_flops / (ms_e2e * 1e-3) / 1e12, unit="TFLOP/s", ms_per_step=ms_e2e,
                        h2d_bytes_per_step=host_x.numel() * 2 * world, d2h_bytes_per_step=host_out.numel() * 2 * world,
                        steps=n),
            "gpu_launches": 9 * chunks * args.steps, "clocks": clocks.summary(),
        }))
    dist.destroy_process_group()


def run_e2e(layer, inputs, wl, args, flops):
    """The user's call path: torch.ops.paired_nvfp4.* with freshly allocated outputs; each step copies the
    activations in from pinned host memory and the layer output back out."""
    import torch
    ops = torch.ops.paired_nvfp4
    x = inputs["x"]
    host_x = x.cpu().pin_memory()
    dev_x = torch.empty_like(x)
    E, H, I, cap = layer.E, layer.H, layer.I, layer.cap
    out1 = torch.zeros((E, cap, 2 * I), dtype=torch.bfloat16, device=x.device)
    out2 = torch.zeros((E, cap, H), dtype=torch.bfloat16, device=x.device)
    w = layer.weights[0]
    name = layer.cabi.group_mm_config_names()[layer.cfg]
    routed = layer.flat_tok is not None
    if routed:   # the step ends with the combine: out[t] = sum_j w[t, j] * expert row of routing (t, j)
        T, topk = layer.router_w.shape
        route_dest = torch.where(layer.dest == E * cap, torch.full_like(layer.dest, -1), layer.dest)
        route_dest = route_dest.to(torch.int32).view(T, topk).contiguous()
        final = torch.zeros((T, H), dtype=torch.bfloat16, device=x.device)
        host_out = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
    else:
        final = out2
        host_out = torch.empty((E, cap, H), dtype=torch.bfloat16).pin_memory()

    def finish():
        if routed:
            ops.moe_finalize(final, out2, route_dest, layer.router_w)
        host_out.copy_(final, non_blocking=True)

    def one():
        dev_x.copy_(host_x, non_blocking=True)
        if layer.flat_tok is None:
            b1, s1 = ops.quant_act(dev_x, layer.g1, layer.counts, 2 * I)
        else:
            b1, s1 = ops.scatter_quant_act(dev_x, layer.flat_tok, layer.dest, layer.topk_w, layer.g1, layer.counts, cap)
        if layer.fused:
            b2, s2 = ops.group_mm_swiglu_quant(w["a13"], w["e13"], w["s13"], b1, s1, layer.al1, layer.counts, layer.g2,
                                               2 * I, H, layer.fused_cfg, layer.cluster_m, 1)
        else:
            ops.group_mm(out1, w["a13"], w["e13"], w["s13"], b1, s1, layer.al1, layer.counts, 2 * I, H, layer.cfg,
                         layer.cluster_m, 1)
            b2, s2 = ops.silu_mul_quant_act(out1, layer.g2, layer.counts, H)
        ops.group_mm(out2, w["a2"], w["e2"], w["s2"], b2, s2, layer.al2, layer.counts, H, I, layer.cfg, layer.cluster_m, 1)
        finish()
        torch.cuda.synchronize()

    for _ in range(3):
        one()
    # The launches are fixed-shape and read counts on the device, so the step (copy in, layer, copy out) is
    # captured once in a CUDA graph, as a serving loop would, and replayed; every replay re-reads the pinned
    # host buffer and rewrites the host result.
    mode = "cuda graph replay"
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                dev_x.copy_(host_x, non_blocking=True)
                if layer.flat_tok is None:
                    b1, s1 = ops.quant_act(dev_x, layer.g1, layer.counts, 2 * I)
                else:
                    b1, s1 = ops.scatter_quant_act(dev_x, layer.flat_tok, layer.dest, layer.topk_w, layer.g1, layer.counts, cap)
                if layer.fused:
                    b2, s2 = ops.group_mm_swiglu_quant(w["a13"], w["e13"], w["s13"], b1, s1, layer.al1, layer.counts,
                                                       layer.g2, 2 * I, H, layer.fused_cfg, layer.cluster_m, 1)
                else:
                    ops.group_mm(out1, w["a13"], w["e13"], w["s13"], b1, s1, layer.al1, layer.counts, 2 * I, H,
                                 layer.cfg, layer.cluster_m, 1)
                    b2, s2 = ops.silu_mul_quant_act(out1, layer.g2, layer.counts, H)
                ops.group_mm(out2, w["a2"], w["e2"], w["s2"], b2, s2, layer.al2, layer.counts, H, I, layer.cfg,
                             layer.cluster_m, 1)
                finish()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()

        def run():
            graph.replay()
            torch.cuda.synchronize()
        check = host_out.clone()
        host_out.zero_()
        run()
        assert torch.equal(host_out, check), "graph replay does not reproduce the eager step"
    except Exception as exc:   # capture unavailable: time the eager calls
        mode = f"eager calls (graph capture failed: {type(exc).__name__})"
        run = one
    n = max(5, min(args.steps, 200))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3) / n
    return dict(value=flops / (ms * 1e-3) / 1e12, unit="TFLOP/s", ms_per_step=ms,
                h2d_bytes_per_step=host_x.numel() * 2, d2h_bytes_per_step=host_out.numel() * 2,
                steps=n, tile_config=name, mode=mode)


def run_reference_arm(args, wl_name, wl, rank):
    """The reference's CPU implementation of the path (reference.py semantics, restated in numpy by
    the oracle) on the host cores: each step is a bounded sample of the workload."""
    if rank != 0:
        return
    from oracle import paired_nvfp4_oracle as orc
    H, I = wl["hidden"], wl["inter"]
    rng = np.random.default_rng(wl["seed"])
    rows = 16 if wl["routing"] == "counts" else 64
    m13, m2 = min(2 * I, 1024), min(H, 512)   # a slice of output features of one expert per step
    w13 = orc.prune_paired_4of8((rng.standard_normal((1, m13, H)) * wl["wstd"]).astype(np.float32))
    w2 = orc.prune_paired_4of8((rng.standard_normal((1, m2, I)) * wl["wstd"]).astype(np.float32))
    p13, s13, _ = orc.quantize_weight(w13)
    p2, s2, _ = orc.quantize_weight(w2)
    x = orc.f32_to_bf16_bits(rng.standard_normal((1, rows, H)).astype(np.float32))
    x2 = orc.f32_to_bf16_bits(rng.standard_normal((1, rows, 2 * I)).astype(np.float32))
    cnt = np.array([rows], np.int32)
    one = np.ones(1, np.float32)
    flops_step = 2.0 * rows * (m13 * H + m2 * I)

    def step():
        b1, _, sfb1 = orc.quant_act(x, one, cnt)
        orc.group_mm(orc.dequantize_weight(p13, s13), b1, sfb1, one, cnt)
        b2, _, sfb2, _ = orc.silu_mul_quant_act(x2, one, cnt)
        orc.group_mm(orc.dequantize_weight(p2, s2), b2, sfb2, one, cnt)

    for _ in range(min(args.warmup, 3)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    ms = dt / args.steps * 1e3
    value = flops_step / (ms * 1e-3) / 1e12
    sample = (f"per step: one expert, {rows} rows, {m13} of {2 * I} gate_up features and {m2} of {H} down features: "
              "numpy oracle quantizers + weight dequantisation + fp32 matmuls")
    print(json.dumps({
        "impl": "reference", "metric": "moe_expert_ffn_group_mm_dense_equiv_tflops", "value": value,
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": min(args.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": f"{wl_name}: {wl['desc']}", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


if __name__ == "__main__":
    main()
