"""GPU parity: group_mm against the oracle's fp32 dequantised matmul.  Bar: relative Frobenius
error <= 5e-3 on the valid rows (the only error sources are fp32 accumulation order and the final
bf16 rounding), and every row at or past counts[e] keeps the caller's bytes."""
import numpy as np
import pytest
import torch

from oracle import paired_nvfp4_oracle as orc
from helpers import bf16_tensor, u8, dev, make_acts, make_weights

pytestmark = pytest.mark.gpu

REL_FROB_TOL = 5e-3
SENTINEL = -12352.0   # the reference's -12345 sentinel as bf16 stores it


@pytest.fixture(scope="module")
def pnk():
    import paired_nvfp4_kernels
    return paired_nvfp4_kernels


def run_case(pnk, E, M, K, max_n, counts, config_id, seed, wscale=1.0, gscale=None, alphas=None, cluster=None):
    ops = torch.ops.paired_nvfp4
    packed, sf, w_dq = make_weights(E, M, K, seed, wscale)
    x = make_acts(E, max_n, K, seed + 1)
    cnt = np.asarray(counts, np.int32)
    g = np.ones(1, np.float32) if gscale is None else np.asarray(gscale, np.float32)
    al = np.linspace(0.5, 2.0, E).astype(np.float32) if alphas is None else np.asarray(alphas, np.float32)
    a_comp, e_meta, sfa = ops.compress(dev(packed), dev(sf), K)
    b_act, sfb = ops.quant_act(bf16_tensor(x), dev(g), dev(cnt), M)
    out = torch.full((E, max_n, M), SENTINEL, dtype=torch.bfloat16, device="cuda")
    name = pnk.group_mm_configs()[config_id]
    cm, cn = cluster or pnk.valid_clusters(name)[0]
    ops.group_mm(out, a_comp, e_meta, sfa, b_act, sfb, dev(al), dev(cnt), M, K, config_id, cm, cn)
    torch.cuda.synchronize()
    from paired_nvfp4_kernels import ops as pyops
    assert pyops.group_mm_device_status() == 0
    got = out.float().cpu().numpy()
    ob, valid, osfb = orc.quant_act(x, g, cnt)
    assert np.array_equal(u8(sfb), osfb)
    want = orc.group_mm(w_dq, ob, osfb, al, cnt, sentinel=SENTINEL)
    assert (got[~valid] == SENTINEL).all(), "rows at or past counts[e] were written"
    # the bar holds for every expert on its own, so a wrong small expert cannot hide behind a large right one
    for e in range(E):
        n = int(min(cnt[e], max_n))
        if n > 0:
            rel = orc.rel_frobenius(got[e, :n], want[e, :n])
            assert rel <= REL_FROB_TOL, f"expert {e}: relative Frobenius error {rel:.3e}"
    return got, want, valid


def config_ids():
    return list(range(9))


@pytest.mark.parametrize("config_id", config_ids())
def test_small_single_tile(pnk, config_id):
    run_case(pnk, E=1, M=128, K=256, max_n=32, counts=[32], config_id=config_id, seed=10)


@pytest.mark.parametrize("config_id", config_ids())
def test_zero_count_experts_and_untouched_padding(pnk, config_id):
    # the reference's tests/test_ops.py:121-145 case: counts straddling every tile boundary
    run_case(pnk, E=8, M=512, K=512, max_n=512, counts=[0, 1, 255, 256, 257, 512, 0, 64],
             config_id=config_id, seed=0)


SHAPES = [
    # E, M, K, max_n, counts
    (8, 2048, 1024, 256, "rand"),                 # the reference's CPU-plumbing config
    (2, 130, 320, 70, [70, 3]),                   # M tail, K = 2.5 MMA blocks, K atoms with slop
    (3, 256, 96, 40, [40, 0, 17]),                # K below one MMA block
    (2, 384, 4096, 16, [16, 5]),                  # long K, decode-sized counts
    (4, 1536, 2048, 300, [300, 128, 129, 1]),     # Qwen3 gate_up shape
    (2, 2048, 768, 200, [200, 64]),               # Qwen3 down shape (K = 3 stages)
    (1, 128, 14336, 8, [8]),                      # Mixtral down K
]


@pytest.mark.parametrize("E,M,K,max_n,counts", SHAPES)
@pytest.mark.parametrize("config_id", [0, 1, 5, 7, 8])
def test_shapes(pnk, E, M, K, max_n, counts, config_id):
    if counts == "rand":
        counts = np.random.default_rng(1001).integers(1, max_n + 1, E)
    run_case(pnk, E, M, K, max_n, counts, config_id, seed=E + M + K)


@pytest.mark.parametrize("config_id", [0, 1, 5, 8])
def test_many_long_tiles_per_cta(pnk, config_id):
    # more tiles than SMs, each tile's K loop longer than the shared-memory stage ring: every CTA
    # walks several tiles and the pipeline barriers go through many phases
    run_case(pnk, E=4, M=1024, K=2048, max_n=2048, counts=[2048, 1900, 2047, 1500], config_id=config_id, seed=77,
             wscale=0.05)


@pytest.mark.parametrize("config_id", [0, 1])
@pytest.mark.parametrize("K", [768, 2048, 3072])
def test_pair_kernels_over_many_ragged_experts(pnk, config_id, K):
    # many experts with ragged counts (some empty, one full, one with a single token) on the pair kernels: more
    # tiles than CTA pairs, M not a multiple of the pair's 256 rows, K loops shorter and longer than the ring
    rng = np.random.default_rng(K)
    counts = rng.integers(0, 601, 28)
    counts[[3, 4, 17]] = 0
    counts[5], counts[6] = 600, 1
    run_case(pnk, E=28, M=768 - 24, K=K, max_n=600, counts=counts.tolist(), config_id=config_id, seed=K, wscale=0.05)


@pytest.mark.parametrize("M", [256, 640 - 8, 1536])
@pytest.mark.parametrize("K", [256, 1280, 3328])
def test_narrow_tail_tiles_against_two_m_units(pnk, M, K):
    # the 256 x 256 pair kernel multiplies an expert's last token tile, when it holds at most 64 rows, against two
    # M units per work item (when no expert can hold more than four token tiles): counts just past a tile boundary
    # (1, 64 rows over), at it, and past the narrow limit (65 over), over one, three (odd: the last item has one unit)
    # and six M units, K loops of one stage, fewer stages than the ring and more; the longest K runs 512-K stages
    # with a short last one
    counts = [257, 320, 321, 256, 64, 1, 512 + 64, 300, 0, 512 + 65]
    for cid in (1, 3) if M == 256 else (1,):   # the pair kernel (and once the single-CTA 256-token kernel beside it)
        run_case(pnk, E=len(counts), M=M, K=K, max_n=640, counts=counts, config_id=cid, seed=M + K, wscale=0.05)


def test_gscale_and_alpha_undo_each_other(pnk):
    E, M, K, max_n = 4, 256, 512, 48
    x_amax = 4.5
    g = np.full(E, 6 * 448 / x_amax, np.float32) * np.array([1, 0.5, 0.25, 2], np.float32)
    got, want, valid = run_case(pnk, E, M, K, max_n, [48, 7, 0, 33], 0, seed=5, wscale=0.02, gscale=g, alphas=1.0 / g)
    assert np.abs(want[valid]).max() > 0.01


def test_every_tactic_matches_default(pnk):
    E, M, K, max_n = 3, 384, 512, 150
    base, _, valid = run_case(pnk, E, M, K, max_n, [150, 31, 97], 0, seed=3)
    for cid, cm, cn in pnk.all_tactics():
        got, _, _ = run_case(pnk, E, M, K, max_n, [150, 31, 97], cid, seed=3, cluster=(cm, cn))
        assert np.allclose(got[valid], base[valid], atol=1e-2, rtol=1e-2)


def test_pair_kernels_on_odd_tile_counts(pnk):
    # M = 3 and 5 tiles of 128 rows: the second CTA of the last pair has no tile of its own and must store nothing
    for cid in (0, 1, 4, 6):
        run_case(pnk, E=3, M=384, K=768, max_n=200, counts=[200, 0, 77], config_id=cid, seed=21)
        run_case(pnk, E=2, M=640 - 8, K=512, max_n=96, counts=[96, 33], config_id=cid, seed=22)


ROW_MAP_CASES = [
    # E, M, K, max_n, counts, config ids
    (3, 384, 768, 200, [200, 0, 77], (0, 1, 3, 5, 8)),       # wide kernels, single CTA and pairs, odd tile count
    (2, 250, 512, 300, [300, 150], (1, 2)),                  # 256-token tiles (two chunks per group); M tail
    (4, 768, 512, 330, [300, 257, 320, 64], (1,)),           # narrow tail tiles against two M units (three units: odd)
    (4, 512, 2048, 16, [16, 0, 3, 9], (7,)),                 # narrow kernel, K split across CTAs
    (2, 202, 1024, 32, [32, 20], (7,)),                      # narrow kernel, scalar store path (M % 8 != 0)
]


@pytest.mark.parametrize("E,M,K,max_n,counts,cids", ROW_MAP_CASES)
def test_group_mm_rows_permutes_the_output(pnk, E, M, K, max_n, counts, cids):
    """group_mm_rows == group_mm followed by a row permutation: kept rows land where the map says, bit for bit;
    rows mapped to -1 and rows no token maps to keep the caller's bytes."""
    ops = torch.ops.paired_nvfp4
    packed, sf, _ = make_weights(E, M, K, 31)
    x = make_acts(E, max_n, K, 32)
    cnt = np.asarray(counts, np.int32)
    a_comp, e_meta, sfa = ops.compress(dev(packed), dev(sf), K)
    b_act, sfb = ops.quant_act(bf16_tensor(x), dev(np.ones(1, np.float32)), dev(cnt), M)
    al = dev(np.linspace(0.5, 2.0, E).astype(np.float32))
    rng = np.random.default_rng(33)
    rows = (E * max_n + 5 + 3) // 4 * 4                       # a multiple of four: the parts form cuts it in four
    to = rng.permutation(rows)[:E * max_n].astype(np.int32)
    to[rng.random(E * max_n) < 0.1] = -1                      # some kept rows are not wanted
    live = (np.arange(max_n)[None, :] < cnt[:, None]).reshape(-1)
    to_dev = dev(np.where(live, to, np.int32(2 ** 30)))       # entries of rows past counts[e] are never read
    for cid in cids:
        name = pnk.group_mm_configs()[cid]
        cm, cn = pnk.valid_clusters(name)[0]
        plain = torch.full((E, max_n, M), SENTINEL, dtype=torch.bfloat16, device="cuda")
        ops.group_mm(plain, a_comp, e_meta, sfa, b_act, sfb, al, dev(cnt), M, K, cid, cm, cn)
        out = torch.full((rows, M), SENTINEL, dtype=torch.bfloat16, device="cuda")
        ops.group_mm_rows(out, to_dev, a_comp, e_meta, sfa, b_act, sfb, al, dev(cnt), M, K, cid, cm, cn)
        torch.cuda.synchronize()
        want = torch.full((rows, M), SENTINEL, dtype=torch.bfloat16, device="cuda")
        keep = torch.from_numpy(live & (to >= 0)).cuda()
        want[torch.from_numpy(to).cuda().long()[keep]] = plain.view(E * max_n, M)[keep]
        assert torch.equal(out, want), name
        # the same output cut into four separately allocated buffers
        parts = [torch.full((rows // 4, M), SENTINEL, dtype=torch.bfloat16, device="cuda") for _ in range(4)]
        ops.group_mm_rows_parts(parts, to_dev, a_comp, e_meta, sfa, b_act, sfb, al, dev(cnt), M, K, cid, cm, cn)
        torch.cuda.synchronize()
        assert torch.equal(torch.cat(parts), want), name + " (parts)"
    from paired_nvfp4_kernels import ops as pyops
    assert pyops.group_mm_device_status() == 0


SPLIT_CASES = [
    # E, M, K, max_n, counts: decode-sized problems, where the K stages of all tiles are dealt evenly to the SMs
    (2, 256, 4096, 16, [16, 5]),                  # 4 tiles x 8 stages over 32 CTAs: every CTA gets one stage of a tile
    (8, 512, 2048, 8, [0, 0, 0, 7, 0, 0, 0, 0]),  # one active expert: most CTAs get an empty range
    (1, 128, 2176, 32, [32]),                     # K = 4 stages + a short tail stage that is a unit of its own
    (3, 384, 14336, 16, [16, 1, 9]),              # long K, tiles cut at arbitrary stages
    (8, 1024, 7168, 1, [0, 0, 0, 1, 0, 0, 0, 0]),   # one token on one expert (an expert-parallel decode rank)
]


@pytest.mark.parametrize("E,M,K,max_n,counts", SPLIT_CASES)
def test_split_k_matches_oracle_and_unsplit(pnk, E, M, K, max_n, counts):
    """Through the operators the split is on (they keep a workspace per stream); through the C ABI with no
    workspace it is off.  Both must meet the bar; twice in a row, to show the counters return to zero."""
    from paired_nvfp4_kernels import _cabi
    ops = torch.ops.paired_nvfp4
    got_a, want, valid = run_case(pnk, E, M, K, max_n, counts, 7, seed=31)
    got_b, _, _ = run_case(pnk, E, M, K, max_n, counts, 7, seed=31)
    assert np.array_equal(got_a, got_b), "the split result must not depend on timing"
    # the same launch without a workspace
    packed, sf, _ = make_weights(E, M, K, 31, 1.0)
    x = make_acts(E, max_n, K, 32)
    cnt = np.asarray(counts, np.int32)
    al = np.linspace(0.5, 2.0, E).astype(np.float32)
    a_comp, e_meta, sfa = ops.compress(dev(packed), dev(sf), K)
    b_act, sfb = ops.quant_act(bf16_tensor(x), dev(np.ones(1, np.float32)), dev(cnt), M)
    out = torch.full((E, max_n, M), SENTINEL, dtype=torch.bfloat16, device="cuda")
    al_t, cnt_t = dev(al), dev(cnt)
    _cabi.check(_cabi.lib.pnv_group_mm(out.data_ptr(), a_comp.data_ptr(), e_meta.data_ptr(), sfa.data_ptr(),
                                       b_act.data_ptr(), sfb.data_ptr(), al_t.data_ptr(), cnt_t.data_ptr(), E, M, K, max_n,
                                       7, 1, 1, 0, 1, None, 0, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    plain = out.float().cpu().numpy()
    assert (plain[~valid] == SENTINEL).all()
    for e in range(E):
        n = int(cnt[e])
        if n:
            assert orc.rel_frobenius(plain[e, :n], want[e, :n]) <= REL_FROB_TOL
            # split and unsplit differ only in the order of the fp32 sum: at most an ulp of bf16 here and there
            assert orc.rel_frobenius(got_a[e, :n], plain[e, :n]) <= 4e-3


def test_bounded_wait_gives_up_and_reports(pnk):
    """The give-up path of the kernels' bounded waits, with nothing in flight: a wait on a barrier nobody
    arrives at must return, leave its code in the status word, and leave the context usable."""
    import ctypes
    from paired_nvfp4_kernels import _cabi, ops as pyops
    assert pyops.group_mm_device_status() == 0
    gave_up = ctypes.c_int(-1)
    _cabi.check(_cabi.lib.pnv_selftest_bounded_wait(ctypes.byref(gave_up)))
    assert gave_up.value == 1
    assert pyops.group_mm_device_status() == 99
    assert pyops.group_mm_device_status() == 0          # reading clears the word
    run_case(pnk, E=1, M=128, K=256, max_n=32, counts=[32], config_id=2, seed=10)   # the context still works


def test_argument_checks(pnk):
    ops = torch.ops.paired_nvfp4
    E, M, K, max_n = 1, 128, 256, 16
    packed, sf, _ = make_weights(E, M, K, 1)
    a_comp, e_meta, sfa = ops.compress(dev(packed), dev(sf), K)
    cnt = dev(np.array([16], np.int32))
    b_act, sfb = ops.quant_act(bf16_tensor(make_acts(E, max_n, K, 2)), dev(np.ones(1, np.float32)), cnt, M)
    al = dev(np.ones(1, np.float32))
    out = torch.zeros(E, max_n, 2 * M, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="compress"):
        ops.group_mm(out, a_comp, e_meta, sfa, b_act, sfb, al, cnt, 2 * M, K)
    out = torch.zeros(E, max_n, M, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="even cluster_m"):
        ops.group_mm(out, a_comp, e_meta, sfa, b_act, sfb, al, cnt, M, K, 0, 1, 1)
    with pytest.raises(RuntimeError, match="config_id"):
        ops.group_mm(out, a_comp, e_meta, sfa, b_act, sfb, al, cnt, M, K, 99, 2, 1)
    with pytest.raises(RuntimeError, match="powers of two"):
        ops.group_mm(out, a_comp, e_meta, sfa, b_act, sfb, al, cnt, M, K, 2, 3, 1)
