// group_mm: out[e, t, :] = bf16(alpha[e] * W[e] * x[e, t, :]) for t < counts[e], with W stored
// paired-4:8 sparse NVFP4 (a_comp + e_meta + sfa) and x stored NVFP4 (b_act + sfb).
//
// Persistent kernels, one CTA per SM.  group_mm_kernel (this file) runs the 16- and 32-token tiles of
// decode-sized problems (max_n <= 32); group_mm_wide_kernel (group_mm_wide.cuh) the 64- to 256-token
// tiles, on one CTA per tile ("1sm" variants) or on a CTA pair per tile ("2sm" variants).
// Narrow kernel, four warp roles (6 + ISSUERS warps):
//   warp 0 (one lane)  tile producer: per K stage, the TMA tile loads of the compressed weights and
//                      of the activations (one tensor map each covers every expert; 128-byte swizzle)
//   warp 1 (two lanes) side producer: plain bulk copies of the metadata atoms and of the SFA / SFB
//                      scale atoms, which sit in global memory in exactly the shape tcgen05.cp
//                      consumes and so need no tensor map;
//   ISSUERS warps      MMA issuers (one lane each): issuer j owns a fixed slice of every stage's
//   (one lane each)    128-K blocks.  It copies their metadata and scales into tensor memory
//                      (tcgen05.cp), issues one tcgen05.mma.sp block-scaled instruction
//                      (128 x TILE_N x 128) per block into its own partial accumulator, and commits:
//                      to the stage's "empty" barrier, and after the tile's last stage to the
//                      accumulator's "full" barrier.  A tcgen05 operation holds its issuing thread
//                      for about as long as it executes (MMA 66-160 cycles, copy 35-50) and the
//                      thread's own instructions in between add to that, so with narrow tiles a
//                      single issuer, not memory, would bound the kernel; issuers in different
//                      warps overlap.
//   last 4 warps       epilogue: tcgen05.ld the partial accumulators 32 token columns at a time, add
//                      them, scale by alpha[e], round to bf16, transpose through shared memory and
//                      store 16 bytes per thread, 256 contiguous bytes per output row; or, in the
//                      fused variant, apply the gated activation and write GEMM2's codes and scales.
// Accumulators are double buffered, so the epilogue of one tile overlaps the main loop of the next.
//
// Tile schedule: every role walks the same list on its own, derived on the device from
// counts[]: experts in order, each contributing ceil(M/128) * ceil(counts[e]/TILE_N) tiles
// (M tile fastest); CTA b takes tiles b, b + grid, ...  No host read of counts, no scheduler
// state in global memory: the launch is fixed-shape and safe to capture in a CUDA graph.
//
// Every mbarrier wait is bounded; a wait that gives up records a code in g_status, and every role
// leaves its loop and meets at the final barrier, where tensor memory is released.
#include <cuda.h>

#include <algorithm>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace pnv {
namespace {

__device__ int g_status = 0;

constexpr int kTileM = 128;
constexpr int kEpilogueThreads = 128;
constexpr int kTmemCols = 512;
constexpr int kColE = 448;                   // tensor-memory columns: metadata (up to 16)
constexpr int kColSfa = 464;                 //   weight scales (4 per K-block)
constexpr int kColSfb = 480;                 //   activation scales (4 or 8 per K-block)
constexpr int kOutRow = kTileM + 8;          // padded row of the epilogue transpose buffer (bank spread)
constexpr int kOutStageBytes = 2 * 32 * kOutRow * 2;   // 2 x [32 token columns][136] bf16
constexpr int kMaxExperts = 2048;            // bounds the shared-memory copy of counts
constexpr int kSmemLimit = 227 * 1024;

enum Status : int {
  kOk = 0, kProducerEmptyTimeout = 1, kMmaFullTimeout = 2, kMmaAccTimeout = 3, kEpilogueTimeout = 4,
  kSideProducerTimeout = 5, kMmaScaleTimeout = 6, kScaleLoaderTimeout = 7, kSelfTestTimeout = 99
};

template <int TILE_N, int STAGE_K, int ISSUERS>
struct Cfg {
  static_assert(TILE_N == 16 || TILE_N == 32 || TILE_N == 64 || TILE_N == 128 || TILE_N == 256,
                "tile widths: 16 and 32 (single token tile only), 64, 128, 256");
  static_assert(ISSUERS == 1 || ISSUERS == 2 || ISSUERS == 4, "MMA issuer warps: 1, 2 or 4");
  static constexpr int kThreads = (6 + ISSUERS) * 32;
  static constexpr int kFirstEpilogueWarp = 2 + ISSUERS;
  static_assert(STAGE_K == 256 || STAGE_K == 512, "stage depths: 256, 512");
  static constexpr int kAtoms = STAGE_K / 128;            // MMA K-blocks per stage
  static constexpr int kARowBytes = STAGE_K / 4;          // compressed weight bytes per row per stage
  static constexpr int kABytes = kTileM * kARowBytes;
  static constexpr uint32_t kASwizzle = STAGE_K == 512 ? 2 : 4;   // descriptor code: 128-B / 64-B swizzle
  static constexpr int kBBoxes = STAGE_K / 256;           // 128-byte-wide activation boxes per stage
  static constexpr int kBBoxBytes = TILE_N * 128;
  static constexpr int kBBytes = kBBoxes * kBBoxBytes;
  static constexpr int kEAtoms = STAGE_K / 256;
  static constexpr int kEBytes = 2048 * kEAtoms;
  static constexpr int kSfaBytes = 512 * kAtoms;
  static constexpr int kSfbRowAtoms = TILE_N > 128 ? 2 : 1;
  static constexpr int kSfbBytes = kSfaBytes * kSfbRowAtoms;
  static constexpr int kStageBytes = kABytes + kBBytes + kEBytes + kSfaBytes + kSfbBytes;
  static constexpr int kFixedBytes = 1024 + kOutStageBytes + 256 + 4 * kMaxExperts;
  static constexpr int kStages = (kSmemLimit - kFixedBytes) / kStageBytes;
  static constexpr int kAccStages = TILE_N == 256 ? 1 : 2;
  static constexpr int kSfbColsPerAtom = 4 * kSfbRowAtoms;
  static constexpr int kAtomsPerIssuer = kAtoms / ISSUERS;          // K-blocks of a stage per issuer
  static constexpr int kEAtomsPerIssuer = kAtomsPerIssuer >= 2 ? kAtomsPerIssuer / 2 : 1;
  static constexpr int kEColsPerIssuer = 4 * kEAtomsPerIssuer;      // private metadata columns
  static_assert(kAtomsPerIssuer >= 1, "more issuers than K-blocks per stage");
  static constexpr int kOffA = 0;
  static constexpr int kOffB = kABytes;
  static constexpr int kOffE = kOffB + kBBytes;
  static constexpr int kOffSfa = kOffE + kEBytes;
  static constexpr int kOffSfb = kOffSfa + kSfaBytes;
  static_assert(kStageBytes % 1024 == 0, "stage buffers must keep 1024-byte alignment");
  static_assert(kStages >= 2, "not enough shared memory for a pipeline");
  static_assert(kAccStages * ISSUERS * TILE_N <= kColE, "accumulators overlap the metadata columns");
  static_assert(kColE + kEColsPerIssuer * ISSUERS <= kColSfa && kColSfa + 4 * kAtoms <= kColSfb &&
                kColSfb + kSfbColsPerAtom * kAtoms <= kTmemCols, "tensor-memory column map overflows");
};

struct Params {
  const uint8_t* e_meta;
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* alphas;
  const int* counts;
  __nv_bfloat16* out;
  // plain epilogue: token row (e, n) is written to output row row_map[e * max_n + n] of a [rows, M] output,
  // and not at all where the map is negative; nullptr = row e * max_n + n
  const int* row_map;
  RowParts out_parts;  // with a row map: the output rows spread over several buffers (n = 0: all in `out`)
  int E, M, K, max_n;
  int n_mt;          // ceil(M / 128)
  int k_stages;      // ceil(K / STAGE_K)
  int n_kt;          // scale K-atoms per row = MMA K-blocks = ceil(K / 128)
  int e_k_atoms;     // metadata atoms along K = ceil(K / 256)
  int e_m_atoms;     // metadata atoms along M = n_mt
  int sfb_rt;        // scale row-atoms per expert in sfb = ceil(max_n / 128)
  int stages;        // pipeline depth in use (<= Cfg::kStages)
  int b_4d;          // map_b is the 4-D view [E][K/256][max_n][128 B] and one copy fetches a whole stage
  int prod_lanes;    // wide kernel: lanes of each producer warp that issue copies side by side
  int b_tail;        // wide kernel: a second activation map with a 64-token box exists (narrow tail tiles)
  // narrow kernel, split K (nullptr = every tile on one CTA): per-tile arrival counters (all zero before and
  // after a launch) followed by two partial-accumulator slots per CTA
  int* split_counters;
  float* split_partials;
  // fused SwiGLU + requantise epilogue (kFused kernels): GEMM2's operands instead of a bf16 output
  uint8_t* f_b_out;        // [E, max_n, N/2] e2m1 codes, N = M / 2
  uint8_t* f_sfb_out;      // swizzled scales for (max_n, N), pre-filled with 0x38
  const float* f_gscale;   // GEMM2 activation global scale, [E] or [1]
  int f_gpe;
  int f_n;                 // N
  int f_n_kt;              // scale K-atoms of the N-wide output
  GatedAct f_act;
};

// Where output row `to` of a row-mapped launch starts.
__device__ __forceinline__ __nv_bfloat16* mapped_row(const Params& p, long long to) {
  if (p.out_parts.n == 0) return p.out + to * p.M;
  return reinterpret_cast<__nv_bfloat16*>(part_row(p.out_parts, to, 2LL * p.M));
}

// The walk over (expert, n tile, m tile) shared by all roles.
struct TileWalk {
  const int* cnt;    // shared-memory copy of counts, clamped to [0, max_n]
  int E, n_mt, e;
  long long base;    // first tile index of expert e
  long long tiles_e;
  template <int TILE_N>
  __device__ void init(const int* s_counts, int E_, int n_mt_) {
    cnt = s_counts; E = E_; n_mt = n_mt_; e = 0; base = 0;
    tiles_e = (long long)n_mt * ceil_div_i(cnt[0], TILE_N);
  }
  template <int TILE_N>
  __device__ bool seek(long long t, int& mt, int& nt) {
    while (t >= base + tiles_e) {
      base += tiles_e;
      if (++e >= E) return false;
      tiles_e = (long long)n_mt * ceil_div_i(cnt[e], TILE_N);
    }
    // an expert's own tile count fits 32 bits (its output alone would otherwise exceed the device)
    const unsigned local = (unsigned)(t - base);
    nt = (int)(local / (unsigned)n_mt);
    mt = (int)(local - (unsigned)nt * (unsigned)n_mt);
    return true;
  }
};

// Narrow kernel: the work of one CTA as a list of units (tile, K stages [ks0, ks1)).
//   unsplit   CTA b takes whole tiles b, b + grid, ...
//   split K   the K stages of all tiles, laid end to end, are cut into `grid` equal ranges; CTA b takes range b, so
//             a tile whose stages straddle a cut is multiplied by two or more CTAs.  With few tiles per SM (a
//             decode step with few active experts) that fills every SM and evens out the tail wave.  A partial
//             unit leaves its fp32 accumulator in a slot of the workspace (a CTA has at most two: the head of its
//             range finishing an earlier tile, slot 2b, and the tail starting a later one, slot 2b + 1) and bumps
//             the tile's arrival counter; whichever CTA arrives last adds the tile's slots in K order, so the sum
//             does not depend on timing, and runs the ordinary epilogue.  Nobody waits for anybody.
struct UnitWalk {
  TileWalk tw;
  bool split;
  unsigned ksn, grid;
  // split: K stages of all tiles (the host bounds it below 2^31), and the cut: the first `rem` CTAs take
  // `quot` + 1 stages, the others `quot` -- no division per lookup (a lone thread pays hundreds of cycles for one)
  unsigned total, quot, rem;
  unsigned pos, hi;  // split: this CTA's range; unsplit: pos is the next tile
  template <int TILE_N>
  __device__ void init(const int* s_counts, int E, int n_mt, int k_stages, long long n_tiles, bool split_) {
    tw.init<TILE_N>(s_counts, E, n_mt);
    split = split_; ksn = (unsigned)k_stages; grid = gridDim.x;
    if (split) {
      total = (unsigned)n_tiles * ksn;
      quot = total / grid;
      rem = total - quot * grid;
      pos = range_lo(blockIdx.x);
      hi = range_lo(blockIdx.x + 1);
    } else {
      total = quot = rem = 0; pos = blockIdx.x; hi = 0;
    }
  }
  __device__ unsigned range_lo(unsigned b) const { return quot * b + min(b, rem); }
  // the CTA whose range holds stage x (x < total)
  __device__ unsigned owner(unsigned x) const {
    const unsigned big = rem * (quot + 1);       // stages held by the CTAs with one extra
    return x < big ? x / (quot + 1) : rem + (x - big) / quot;
  }
  // next unit of this CTA; slot = workspace slot of a partial unit
  template <int TILE_N>
  __device__ bool next(long long& tile, int& mt, int& nt, int& ks0, int& ks1, int& slot) {
    if (!split) {
      if (!tw.seek<TILE_N>(pos, mt, nt)) return false;
      tile = pos; ks0 = 0; ks1 = (int)ksn; slot = 0;
      pos += grid;
      return true;
    }
    if (pos >= hi) return false;
    const unsigned t = pos / ksn;
    tile = t;
    ks0 = (int)(pos - t * ksn);
    ks1 = (int)min(ksn, (unsigned)ks0 + (hi - pos));
    slot = 2 * (int)blockIdx.x + (pos == range_lo(blockIdx.x) ? 0 : 1);
    tw.seek<TILE_N>(tile, mt, nt);     // inside the list by construction
    pos += (unsigned)(ks1 - ks0);
    return true;
  }
};

__device__ __forceinline__ void epilogue_bar_sync() {
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

template <int TILE_N, int STAGE_K, int ISSUERS, bool kFused>
__global__ void __launch_bounds__((6 + ISSUERS) * 32, 1)
group_mm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const Params p) {
  using C = Cfg<TILE_N, STAGE_K, ISSUERS>;
  constexpr int kThreads = C::kThreads;
  constexpr int kFirstEpilogueWarp = C::kFirstEpilogueWarp;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  __nv_bfloat16* s_out = reinterpret_cast<__nv_bfloat16*>(smem + C::kStages * C::kStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes + kOutStageBytes);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* acc_full = empty_bar + C::kStages;
  uint64_t* acc_empty = acc_full + C::kAccStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + C::kAccStages);
  int* s_counts = reinterpret_cast<int*>(smem + C::kStages * C::kStageBytes + kOutStageBytes + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- setup that does not depend on the previous kernel ---------------------------------------
  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    // arrivals on a stage's full barrier: the tile producer and the two bulk-copy lanes
    for (int s = 0; s < C::kStages; ++s) { ptx::mbar_init(full_bar + s, 3); ptx::mbar_init(empty_bar + s, ISSUERS); }
    for (int a = 0; a < C::kAccStages; ++a) {
      ptx::mbar_init(acc_full + a, ISSUERS);
      ptx::mbar_init(acc_empty + a, kEpilogueThreads);
    }
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  // counts (and everything else the producer kernels wrote) may only be read after this point
  pdl_wait();
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < p.E; i += kThreads) s_counts[i] = max(0, min(p.counts[i], p.max_n));
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // every thread counts the tiles of the launch (the split schedule is cut from their total)
  long long n_tiles = 0;
  if (p.split_counters != nullptr) {
    for (int e = lane; e < p.E; e += 32) n_tiles += (long long)p.n_mt * ceil_div_i(s_counts[e], TILE_N);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) n_tiles += __shfl_xor_sync(0xffffffffu, n_tiles, o);
  }

  // K is split only when whole tiles would leave SMs idle or the last wave thin (fewer than 1.5 tiles per CTA):
  // with more tiles than that the partial sums and their reduction cost more than the imbalance they remove
  // (measured on an 8-expert decode step: 63.5 / 37.1 us split against 58.9 / 35.2 us whole)
  UnitWalk walk;
  walk.init<TILE_N>(s_counts, p.E, p.n_mt, p.k_stages, n_tiles,
                    p.split_counters != nullptr && 2 * n_tiles < 3LL * (long long)gridDim.x);
  long long tile;
  int mt, nt, ks0, ks1, slot;

  if (warp == 0) {
    // =============================== tile producer (TMA) ===============================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      while (ok && walk.next<TILE_N>(tile, mt, nt, ks0, ks1, slot)) {
        const int e = walk.tw.e;
        const int n0 = nt * TILE_N;
#pragma unroll 1
        for (int ks = ks0; ks < ks1; ++ks) {
          if (!ptx::mbar_wait(empty_bar + stage, phase ^ 1)) {
            atomicExch(&g_status, kProducerEmptyTimeout);
            ok = false;
            break;
          }
          uint8_t* st = stage_base + stage * C::kStageBytes;
          const int k_atoms = min(C::kAtoms, p.n_kt - ks * C::kAtoms);
          const int b_boxes = (k_atoms + 1) / 2;
          // with the 4-D activation map one copy fetches both 256-K chunks of the stage
          ptx::mbar_arrive_expect_tx(full_bar + stage, C::kABytes + (p.b_4d ? C::kBBoxes : b_boxes) * C::kBBoxBytes);
          ptx::tma_load_3d(st + C::kOffA, &map_a, full_bar + stage, ks * C::kARowBytes, mt * kTileM, e);
          if (p.b_4d) {
            ptx::tma_load_4d(st + C::kOffB, &map_b, full_bar + stage, 0, n0, ks * C::kBBoxes, e);
          } else {
            for (int b = 0; b < b_boxes; ++b)
              ptx::tma_load_3d(st + C::kOffB + b * C::kBBoxBytes, &map_b, full_bar + stage,
                               ks * (STAGE_K / 2) + b * 128, n0, e);
          }
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // give copies already in flight time to land before the CTA's shared memory is released
#pragma unroll 1
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =============================== side producer (bulk copies) ===============================
    // two lanes share every stage (lane 0 the metadata atoms, lane 1 the scale atoms), each with its own
    // expect-tx arrival
    if (lane < 2) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      while (ok && walk.next<TILE_N>(tile, mt, nt, ks0, ks1, slot)) {
        const int e = walk.tw.e;
        const int n0 = nt * TILE_N;
        const uint8_t* e_base = p.e_meta + (((long long)e * p.e_k_atoms) * p.e_m_atoms + mt) * 2048;
        const uint8_t* sfa_base = p.sfa + (((long long)e * p.n_mt + mt) * p.n_kt) * 512;
        const uint8_t* sfb_base = p.sfb + (((long long)e * p.sfb_rt + (n0 >> 7)) * p.n_kt) * 512;
        const int sfb_row_atoms = TILE_N > 128 ? min(2, p.sfb_rt - (n0 >> 7)) : 1;
        for (int ks = ks0; ks < ks1; ++ks) {
          if (!ptx::mbar_wait(empty_bar + stage, phase ^ 1)) {
            atomicExch(&g_status, kSideProducerTimeout);
            ok = false;
            break;
          }
          uint8_t* st = stage_base + stage * C::kStageBytes;
          const int k_atoms = min(C::kAtoms, p.n_kt - ks * C::kAtoms);
          const int e_atoms = (k_atoms + 1) / 2;
          const uint32_t sf_bytes = 512u * k_atoms;
          const uint8_t* sfa_src = sfa_base + (long long)ks * C::kAtoms * 512;
          if (lane == 0) {
            ptx::mbar_arrive_expect_tx(full_bar + stage, e_atoms * 2048);
            for (int ea = 0; ea < e_atoms; ++ea)
              ptx::bulk_load(st + C::kOffE + ea * 2048,
                             e_base + (long long)(ks * C::kEAtoms + ea) * p.e_m_atoms * 2048, 2048,
                             full_bar + stage);
          } else {
            ptx::mbar_arrive_expect_tx(full_bar + stage, sf_bytes * (1 + sfb_row_atoms));
            ptx::bulk_load(st + C::kOffSfa, sfa_src, sf_bytes, full_bar + stage);
            for (int ra = 0; ra < sfb_row_atoms; ++ra)
              ptx::bulk_load(st + C::kOffSfb + ra * C::kSfaBytes,
                             sfb_base + ((long long)ra * p.n_kt + ks * C::kAtoms) * 512, sf_bytes,
                             full_bar + stage);
          }
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
#pragma unroll 1
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp < 2 + ISSUERS) {
    // =============================== MMA issuers ===============================
    if (lane == 0) {
      const int issuer = warp - 2;
      constexpr int kPer = C::kAtomsPerIssuer;
      const int ka0 = issuer * kPer;               // this issuer's K-blocks of a stage: [ka0, ka0 + kPer)
      constexpr uint32_t idesc = ptx::mma_sp_nvf4_idesc(TILE_N);
      const uint32_t e_cols = tmem_base + kColE + issuer * C::kEColsPerIssuer;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      while (ok && walk.next<TILE_N>(tile, mt, nt, ks0, ks1, slot)) {
        if (!ptx::mbar_wait(acc_empty + acc, acc_phase ^ 1)) {
          atomicExch(&g_status, kMmaAccTimeout);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (acc * ISSUERS + issuer) * TILE_N;
        // The scales of a 64-wide tile's rows sit 0 or 2 columns into the 128-row atom.  The MMA
        // faults (misaligned address) on an odd column offset, which is why 16- and 32-wide tiles
        // exist only for problems with a single token tile (offset 0).
        const uint32_t sfb_col = tmem_base + kColSfb + (TILE_N < 128 ? ((nt * TILE_N) & 127) >> 5 : 0);
        for (int ks = ks0; ks < ks1; ++ks) {
          if (!ptx::mbar_wait(full_bar + stage, phase)) {
            atomicExch(&g_status, kMmaFullTimeout);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t st = ptx::smem_u32(stage_base + stage * C::kStageBytes);
          const int k_atoms = min(C::kAtoms, p.n_kt - ks * C::kAtoms);
          if (ka0 < k_atoms) {
            // metadata atoms covering this issuer's K-blocks, into its private columns
#pragma unroll
            for (int i = 0; i < C::kEAtomsPerIssuer; ++i) {
              const int ea = ka0 / 2 + i;
              if (2 * ea < k_atoms)
                ptx::tc_cp_128x128b(e_cols + i * 4, ptx::smem_desc(st + C::kOffE + ea * 2048, 128, 0, 0));
            }
          }
#pragma unroll
          for (int i = 0; i < kPer; ++i) {
            const int ka = ka0 + i;
            if (ka < k_atoms) {
              ptx::tc_cp_32x128b_warpx4(tmem_base + kColSfa + ka * 4,
                                        ptx::smem_desc(st + C::kOffSfa + ka * 512, 128, 0, 0));
#pragma unroll
              for (int ra = 0; ra < C::kSfbRowAtoms; ++ra)
                ptx::tc_cp_32x128b_warpx4(
                    tmem_base + kColSfb + ka * C::kSfbColsPerAtom + ra * 4,
                    ptx::smem_desc(st + C::kOffSfb + ra * C::kSfaBytes + ka * 512, 128, 0, 0));
            }
          }
#pragma unroll
          for (int i = 0; i < kPer; ++i) {
            const int ka = ka0 + i;
            if (ka < k_atoms) {
              const uint64_t a_desc = ptx::smem_desc(st + C::kOffA + ka * 32, 8 * C::kARowBytes, 16, C::kASwizzle);
              const uint64_t b_desc =
                  ptx::smem_desc(st + C::kOffB + (ka >> 1) * C::kBBoxBytes + (ka & 1) * 64, 1024, 16, 2);
              // metadata columns: 2 per K-block inside the atom that holds it
              const uint32_t e_tmem = e_cols + (kPer >= 2 ? i * 2 : (ka & 1) * 2);
              // the first MMA of a unit overwrites this issuer's partial accumulator
              ptx::tc_mma_sp_nvf4(d_tmem, a_desc, b_desc, idesc, ((ks - ks0) | i) != 0 ? 1u : 0u,
                                  tmem_base + kColSfa + ka * 4, sfb_col + ka * C::kSfbColsPerAtom, e_tmem);
            }
          }
          ptx::tc_commit(empty_bar + stage);   // stage reusable once every issuer's MMAs and copies retire
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        ptx::tc_commit(acc_full + acc);        // this issuer's partial accumulator is complete
        if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // =============================== epilogue ===============================
    const int sub = warp & 3;                  // tensor-memory lane quarter this warp may read
    const int ep_tid = threadIdx.x - kFirstEpilogueWarp * 32;
    const int m_local = sub * 32 + lane;       // accumulator row (output feature) held by this thread
    const bool vec_ok = (p.M % 8) == 0;        // 16-byte stores need 16-byte aligned output rows
    int acc = 0;
    uint32_t acc_phase = 0, chunk = 0;
    if (kFused) {
      // Benign fill of GEMM2's scale buffer: every byte the epilogues will not write (rows at or
      // past counts[e], K-block slop) becomes 0x38.  The epilogue warps of all CTAs share the lines;
      // live slots are skipped, so the fill never races with a quantized scale.
      const int KB = p.f_n / kSfBlock;
      const unsigned lines = (unsigned)p.E * p.sfb_rt * p.f_n_kt * 32u;   // < 2^27, checked by the host
      const uint32_t w4 = kBenignSf * 0x01010101u;
#pragma unroll 1
      for (unsigned c = blockIdx.x * kEpilogueThreads + ep_tid; c < lines; c += gridDim.x * kEpilogueThreads) {
        const int rr = (int)(c & 31);
        unsigned a = c >> 5;
        const unsigned a_kt = a / (unsigned)p.f_n_kt;
        const int kt = (int)(a - a_kt * p.f_n_kt);
        const unsigned a_e = a_kt / (unsigned)p.sfb_rt;
        const int r0 = (int)(a_kt - a_e * p.sfb_rt) * 128 + rr;
        const int cnt_e = s_counts[a_e];
        uint8_t* line = p.f_sfb_out + (long long)c * 16;
        if (r0 >= cnt_e) {
          *reinterpret_cast<uint4*>(line) = make_uint4(w4, w4, w4, w4);
        } else {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (r0 + 32 * g >= cnt_e) {
              *reinterpret_cast<uint32_t*>(line + 4 * g) = w4;
            } else {
              for (int j = KB - kt * 4; j < 4; ++j)
                if (j >= 0) line[4 * g + j] = (uint8_t)kBenignSf;
            }
          }
        }
      }
    }
    int* s_last = reinterpret_cast<int*>(tmem_slot + 1);     // "this CTA arrived last at the tile", told to all epilogue threads
    while (walk.next<TILE_N>(tile, mt, nt, ks0, ks1, slot)) {
      const int e = walk.tw.e;
      const int cnt = s_counts[e];
      if (!ptx::mbar_wait(acc_full + acc, acc_phase)) {
        atomicExch(&g_status, kEpilogueTimeout);
        break;
      }
      ptx::tc_fence_after();
      const float alpha = p.alphas[e];
      const int n0 = nt * TILE_N;
      const long long row_e = (long long)e * p.max_n;
      // Issuers whose partial accumulators hold something for this unit.  Every issuer has K-blocks in a full
      // stage; in the (shorter) last stage of a tile the later issuers may have none, and a unit that is just
      // that stage never touched their accumulators.
      const int tail_atoms = p.n_kt - (p.k_stages - 1) * C::kAtoms;
      const int live = ks0 == p.k_stages - 1 ? min(ISSUERS, ceil_div_i(tail_atoms, C::kAtomsPerIssuer)) : ISSUERS;
      const bool partial = ks0 > 0 || ks1 < p.k_stages;
#pragma unroll 1
      for (int c0 = 0; c0 < TILE_N; c0 += 32) {
        if (n0 + c0 >= cnt) break;             // uniform over the four epilogue warps
        uint32_t r[32];
        const uint32_t lane_base = tmem_base + ((uint32_t)(sub * 32) << 16) + c0;
        ptx::tc_ld_32x32(lane_base + (acc * ISSUERS) * TILE_N, r);
        ptx::tc_ld_wait();
#pragma unroll
        for (int j = 1; j < ISSUERS; ++j) {
          if (j < live) {                      // add the other issuers' partial sums
            uint32_t q[32];
            ptx::tc_ld_32x32(lane_base + (acc * ISSUERS + j) * TILE_N, q);
            ptx::tc_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__fadd_rn(__uint_as_float(r[i]), __uint_as_float(q[i])));
          }
        }
        if (partial) {
          // leave this unit's accumulator in its slot ([token column][128 rows] fp32) and count the arrival
          constexpr int kCols = TILE_N < 32 ? TILE_N : 32;
          constexpr int kSlotFloats = kTileM * kCols;
          float* mine = p.split_partials + (long long)slot * kSlotFloats + m_local;
#pragma unroll
          for (int i = 0; i < kCols; ++i) __stcg(mine + i * kTileM, __uint_as_float(r[i]));
          __threadfence();
          epilogue_bar_sync();
          // the CTAs that share this tile, first to last in K
          const unsigned t_lo = (unsigned)tile * walk.ksn, t_hi = t_lo + walk.ksn;
          const unsigned c_first = walk.owner(t_lo), c_last = walk.owner(t_hi - 1);
          const int parts = (int)(c_last - c_first + 1);        // every CTA in between holds stages of the tile
          if (ep_tid == 0) {
            const int before = atomicAdd(p.split_counters + tile, 1);
            *s_last = before == parts - 1 ? 1 : 0;
            if (before == parts - 1) p.split_counters[tile] = 0;     // left zero for the next launch
          }
          epilogue_bar_sync();
          if (*s_last == 0) break;       // another CTA finishes this tile
          __threadfence();
#pragma unroll
          for (int i = 0; i < kCols; ++i) r[i] = 0u;
          for (unsigned d = c_first; d <= c_last; ++d) {
            const int sl = 2 * (int)d + (walk.range_lo(d) >= t_lo ? 0 : 1);     // head of d's range, or its tail
            const float* part = p.split_partials + (long long)sl * kSlotFloats + m_local;
#pragma unroll
            for (int i = 0; i < kCols; ++i)
              r[i] = __float_as_uint(__fadd_rn(__uint_as_float(r[i]), __ldcg(part + i * kTileM)));
          }
        }
        if (kFused) {
          // The weight rows are interleaved in 64-row blocks (32 gate rows, then the 32 matching up
          // rows), so lanes of the even 32-lane quarters hold gates and the odd quarters the ups of
          // the same 32 output features: exactly one quantization block per token.
          __nv_bfloat16* buf = s_out + (chunk & 1) * (32 * kOutRow);
          constexpr int kCols = TILE_N < 32 ? TILE_N : 32;
          __nv_bfloat16 h[kCols];
#pragma unroll
          for (int i = 0; i < kCols; ++i) h[i] = __float2bfloat16_rn(__fmul_rn(alpha, __uint_as_float(r[i])));
          // Every lane parks its values; then the gate lane of a feature finishes the even token
          // columns and the up lane of the same feature the odd ones, each reading its partner's
          // value from shared memory and leaving the product in the gate's slot.  Loads, math and
          // stores are kept in separate passes so the 8 or 16 independent chains overlap.
          const bool is_up = (sub & 1) != 0;
#pragma unroll
          for (int i = 0; i < kCols; ++i) buf[i * kOutRow + m_local] = h[i];
          epilogue_bar_sync();
          constexpr int kHalf = kCols / 2;
          // decode-sized tiles have few pairs per lane: evaluate SiLU directly rather than through the
          // table, whose loads (global memory, mostly L2 with this kernel's shared-memory carve-out) only
          // add latency here
          GatedAct act = p.f_act;
          act.silu_tab = nullptr;
          const int par = is_up ? 1 : 0;
          const int g_row = is_up ? m_local - 32 : m_local;   // the gate's slot, which receives the product
          __nv_bfloat16* col0 = buf + par * kOutRow + g_row;
#pragma unroll 1
          for (int i0 = 0; i0 < kHalf; i0 += 4) {
            float g[4], u[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              g[i] = __bfloat162float(col0[(i0 + i) * 2 * kOutRow]);
              u[i] = __bfloat162float(col0[(i0 + i) * 2 * kOutRow + 32]);
            }
            __nv_bfloat16 y[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) y[i] = __float2bfloat16_rn(gated_act(g[i], u[i], act));
#pragma unroll
            for (int i = 0; i < 4; ++i) col0[(i0 + i) * 2 * kOutRow] = y[i];
          }
          epilogue_bar_sync();
          if (ep_tid < 64) {
            const int i = ep_tid & 31, blk = ep_tid >> 5;
            const int n = n0 + c0 + i;
            if (i < kCols && n < cnt) {
              const uint4* src = reinterpret_cast<const uint4*>(buf + i * kOutRow + blk * 64);
              float f[4][8];
              float amax = 0.f;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                unpack8(src[q], f[q]);
#pragma unroll
                for (int z = 0; z < 8; ++z) amax = fmaxf(amax, fabsf(f[q][z]));
              }
              uint32_t sf_byte;
              float inv;
              block_scale(amax, p.f_gpe ? p.f_gscale[e] : p.f_gscale[0], sf_byte, inv);
              const int kb = mt * 2 + blk;     // 32-feature block of the N-wide output
              const long long row = (long long)e * p.max_n + n;
              *reinterpret_cast<uint4*>(p.f_b_out + row * (p.f_n / 2) + kb * 16) =
                  make_uint4(quant8(f[0], inv), quant8(f[1], inv), quant8(f[2], inv), quant8(f[3], inv));
              p.f_sfb_out[sf_offset(e, n, kb, p.sfb_rt, p.f_n_kt)] = (uint8_t)sf_byte;
            }
          }
          ++chunk;
        } else if (vec_ok) {
          // [token column][feature] tile: 32 rows of 128 bf16; lanes write consecutive features
          __nv_bfloat16* buf = s_out + (chunk & 1) * (32 * kOutRow);
#pragma unroll
          for (int i = 0; i < (TILE_N < 32 ? TILE_N : 32); ++i)
            buf[i * kOutRow + m_local] = __float2bfloat16_rn(__fmul_rn(alpha, __uint_as_float(r[i])));
          epilogue_bar_sync();
          const int col = (ep_tid & 15) * 8;
          const int m = mt * kTileM + col;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int row = (ep_tid >> 4) + 8 * j;
            const int n = n0 + c0 + row;
            if (n < cnt && m < p.M) {
              const long long to = p.row_map ? (long long)p.row_map[row_e + n] : row_e + n;
              if (to >= 0)
                *reinterpret_cast<uint4*>((p.row_map ? mapped_row(p, to) : p.out + to * p.M) + m) =
                    *reinterpret_cast<const uint4*>(buf + row * kOutRow + col);
            }
          }
          ++chunk;
        } else {
          const int m = mt * kTileM + m_local;
          if (m < p.M) {
#pragma unroll
            for (int i = 0; i < (TILE_N < 32 ? TILE_N : 32); ++i) {
              const int n = n0 + c0 + i;
              if (n < cnt) {
                const long long to = p.row_map ? (long long)p.row_map[row_e + n] : row_e + n;
                if (to >= 0)
                  (p.row_map ? mapped_row(p, to) : p.out + to * p.M)[m] = __float2bfloat16_rn(__fmul_rn(alpha, __uint_as_float(r[i])));
              }
            }
          }
        }
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(acc_empty + acc);
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

#include "group_mm_wide.cuh"

// ---- host side -----------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// Tensor maps are pure functions of (base pointer, extents, box, swizzle).  A serving loop calls with
// the same few operand buffers over and over, so the most recent maps are kept and the driver's
// encoder is only called for a new key.  A map holds no reference to the memory it describes: a
// buffer freed and reallocated at the same address with the same shape yields the same map.
struct MapKey {
  const void* base;
  uint64_t row_bytes, rows, experts;
  uint32_t box_rows, box_inner, kind;   // kind: 0 = 3-D tile, 1 = 4-D activation view; swizzle in the high bits
  bool operator==(const MapKey& o) const {
    return base == o.base && row_bytes == o.row_bytes && rows == o.rows && experts == o.experts &&
           box_rows == o.box_rows && box_inner == o.box_inner && kind == o.kind;
  }
};
constexpr int kMapCacheSize = 64;
struct MapCache {
  std::mutex mu;
  MapKey keys[kMapCacheSize];
  CUtensorMap maps[kMapCacheSize];
  int used = 0, next = 0;
};
MapCache g_maps;

template <class Encode>
int cached_map(CUtensorMap* out, const MapKey& key, Encode encode) {
  std::lock_guard<std::mutex> lock(g_maps.mu);
  for (int i = 0; i < g_maps.used; ++i)
    if (g_maps.keys[i] == key) { *out = g_maps.maps[i]; return PNV_OK; }
  if (int rc = encode(out)) return rc;
  const int slot = g_maps.used < kMapCacheSize ? g_maps.used++ : (g_maps.next++ % kMapCacheSize);
  g_maps.keys[slot] = key;
  g_maps.maps[slot] = *out;
  return PNV_OK;
}

// 4-D view of the activations [experts][K/256 chunks][rows][128 B] for K a multiple of 256: one box
// [chunks][box_rows][128 B] is `chunks` consecutive 128-byte-swizzled operand tiles in shared memory.
int make_map_b4(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t experts,
                uint32_t box_rows, uint32_t box_chunks) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(PNV_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  return cached_map(map, MapKey{base, row_bytes, rows, experts, box_rows, box_chunks, 1u}, [&](CUtensorMap* m) {
    cuuint64_t dims[4] = {128, rows, row_bytes / 128, experts};
    cuuint64_t strides[3] = {row_bytes, 128, row_bytes * rows};
    cuuint32_t box[4] = {128, box_rows, box_chunks, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return fail(PNV_ERR_CUDA, "cuTensorMapEncodeTiled (4-D) failed with CUresult %d (row_bytes=%llu rows=%llu)",
                  (int)r, (unsigned long long)row_bytes, (unsigned long long)rows);
    return (int)PNV_OK;
  });
}

// 3-D byte tensor [experts][rows][row_bytes] with a [1][box_rows][box_bytes] box.
int make_map(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t experts,
             uint32_t box_bytes, uint32_t box_rows, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(PNV_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  return cached_map(map, MapKey{base, row_bytes, rows, experts, box_rows, box_bytes, (uint32_t)swz << 8}, [&](CUtensorMap* m) {
    cuuint64_t dims[3] = {row_bytes, rows, experts};
    cuuint64_t strides[2] = {row_bytes, row_bytes * rows};
    cuuint32_t box[3] = {box_bytes, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return fail(PNV_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (row_bytes=%llu rows=%llu)",
                  (int)r, (unsigned long long)row_bytes, (unsigned long long)rows);
    return (int)PNV_OK;
  });
}

// Per kernel instantiation and device, once: opt in to the large dynamic shared-memory carve-out and
// (CTA pairs) allow the cluster launch and ask how many pairs the device runs at the same time.
struct KernelSetup {
  std::once_flag once[64];
  cudaError_t err[64] = {};
  int max_pairs[64] = {};
};

template <class Kernel>
int prepare_kernel(Kernel kernel, KernelSetup& ks, int threads, size_t smem, bool pair, int* max_pairs) {
  int dev = 0;
  PNV_CUDA(cudaGetDevice(&dev));
  PNV_REQUIRE(dev >= 0 && dev < 64, "unexpected CUDA device index %d", dev);
  std::call_once(ks.once[dev], [&] {
    ks.err[dev] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (ks.err[dev] != cudaSuccess || !pair) return;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 148);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    ks.err[dev] = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
    ks.max_pairs[dev] = n;
  });
  if (ks.err[dev] != cudaSuccess)
    return fail(PNV_ERR_CUDA, "group_mm kernel set-up failed: %s", cudaGetErrorString(ks.err[dev]));
  if (max_pairs) *max_pairs = ks.max_pairs[dev];
  return PNV_OK;
}

template <int TILE_N, int STAGE_K, int ISSUERS, bool kFused>
int launch_narrow_impl(const CUtensorMap& map_a, const CUtensorMap& map_b, const Params& p_in, int sm_count, bool pdl,
                       cudaStream_t stream) {
  using C = Cfg<TILE_N, STAGE_K, ISSUERS>;
  Params p = p_in;
  p.stages = C::kStages;
  const size_t smem = 1024 + (size_t)C::kStages * C::kStageBytes + kOutStageBytes + 256 + 4 * (size_t)p.E;
  static_assert(kOutStageBytes % 16 == 0, "barrier block must stay aligned");
  static_assert(8 * (2 * C::kStages + 2 * C::kAccStages) + 16 <= 256, "barrier block overflows its slot");
  static KernelSetup setup;
  if (int rc = prepare_kernel(group_mm_kernel<TILE_N, STAGE_K, ISSUERS, kFused>, setup, C::kThreads, smem, false, nullptr))
    return rc;
  static_assert(TILE_N <= 32, "the split-K epilogue handles one chunk of token columns per tile");
  long long max_units = (long long)p.E * p.n_mt * ceil_div_i(p.max_n, TILE_N);
  if (p.split_counters != nullptr) max_units *= p.k_stages;      // a CTA may get as little as one K stage
  int grid = (int)(max_units < sm_count ? max_units : sm_count);
  if (grid < 1) grid = 1;
  PNV_CUDA(launch_pdl(group_mm_kernel<TILE_N, STAGE_K, ISSUERS, kFused>, dim3(grid), dim3(C::kThreads), smem,
                      stream, pdl, map_a, map_b, p));
  return PNV_OK;
}

template <int TILE_N, int STAGE_K, int ISSUERS>
int launch_narrow(const CUtensorMap& map_a, const CUtensorMap& map_b, Params& p, int sm_count, bool pdl,
                  cudaStream_t stream) {
  if (p.f_b_out != nullptr) return launch_narrow_impl<TILE_N, STAGE_K, ISSUERS, true>(map_a, map_b, p, sm_count, pdl, stream);
  return launch_narrow_impl<TILE_N, STAGE_K, ISSUERS, false>(map_a, map_b, p, sm_count, pdl, stream);
}

// Pipeline depth of a wide-tile launch: what fits beside the epilogue staging, the barriers and the
// counts, capped by the scale-slot ring in tensor memory.
template <class C>
int wide_stages(int experts, bool fused) {
  const int fixed = 1024 + (fused ? C::kFusedOutBytes : C::kPlainOutBytes) + C::kBarrierBytes + 4 * experts;
  int n = std::min(std::min((int)C::kMaxStages, (int)C::kSlots), (kSmemLimit - fixed) / C::kStageBytes);
#ifdef PNV_WIDE_MAX_STAGES      // developer builds: a shallower ring, to see how the time depends on its depth
  n = std::min(n, PNV_WIDE_MAX_STAGES);
#endif
  return n;
}

template <int TILE_N, int STAGE_K, bool kFused, bool kPair, bool kDblTails = false>
int launch_wide_impl(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_b_tail, const Params& p_in,
                     int sm_count, bool pdl, cudaStream_t stream) {
  using C = WideCfg<TILE_N, STAGE_K, kPair, kDblTails>;
  Params p = p_in;
  const int stages = wide_stages<C>(p.E, kFused);
  if (stages < 2)
    return fail(PNV_ERR_INVALID_ARGUMENT, "group_mm: not enough shared memory for a %dx%d pipeline", TILE_N, STAGE_K);
  p.stages = stages;
  p.prod_lanes = stages >= 8 ? 4 : stages >= 4 ? 2 : 1;
  const size_t smem = 1024 + (size_t)stages * C::kStageBytes + (kFused ? C::kFusedOutBytes : C::kPlainOutBytes) +
                      C::kBarrierBytes + 4 * (size_t)p.E;
  static KernelSetup setup;
  int max_pairs = 0;
  if (int rc = prepare_kernel(group_mm_wide_kernel<TILE_N, STAGE_K, kFused, kPair, kDblTails>, setup, C::kThreads, smem, kPair,
                              &max_pairs))
    return rc;
  const long long token_tiles = (long long)p.E * ceil_div_i(p.max_n, TILE_N);
  PNV_REQUIRE(token_tiles * p.n_mt < (1LL << 31), "group_mm: too many tiles for one launch");      // the device walk is 32-bit
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (kPair) {
    PNV_REQUIRE(max_pairs >= 1, "group_mm: this device cannot run a CTA pair of the %dx%d kernel", 2 * kTileM, TILE_N);
    const long long work = token_tiles * ((p.n_mt + 1) / 2);
    long long pairs = std::min<long long>(std::min(max_pairs, sm_count / 2), work);
    if (pairs < 1) pairs = 1;
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 2;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  } else {
    const long long work = token_tiles * p.n_mt;
    long long grid = std::min<long long>(sm_count, work);
    if (grid < 1) grid = 1;
    cfg.gridDim = dim3((unsigned)grid);
  }
  if (pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  PNV_CUDA(cudaLaunchKernelEx(&cfg, group_mm_wide_kernel<TILE_N, STAGE_K, kFused, kPair, kDblTails>, map_a, map_b, map_b_tail, p));
  return PNV_OK;
}

template <int TILE_N, int STAGE_K, bool kPair>
int launch_wide(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_b_tail, Params& p, int sm_count,
                bool pdl, cudaStream_t stream) {
  // Pairs with 256-token tiles: when no expert can hold more than four token tiles, narrow tail tiles are a
  // large enough share of the work for the double-tail-item variant to pay for its overhead on the other items
  // (measured: 256 rows per expert -9 % on the down GEMM, 2048 rows per expert +3 %).
  if constexpr (kPair && TILE_N == 256) {
    if (p.b_tail != 0 && p.max_n <= 4 * TILE_N) {
      if (p.f_b_out != nullptr)
        return launch_wide_impl<TILE_N, STAGE_K, true, kPair, true>(map_a, map_b, map_b_tail, p, sm_count, pdl, stream);
      return launch_wide_impl<TILE_N, STAGE_K, false, kPair, true>(map_a, map_b, map_b_tail, p, sm_count, pdl, stream);
    }
  }
  if (p.f_b_out != nullptr)
    return launch_wide_impl<TILE_N, STAGE_K, true, kPair>(map_a, map_b, map_b_tail, p, sm_count, pdl, stream);
  return launch_wide_impl<TILE_N, STAGE_K, false, kPair>(map_a, map_b, map_b_tail, p, sm_count, pdl, stream);
}

// Tile variants.  The first eight names and ids are the reference's.  "1sm" variants run one CTA per
// 128 x TILE_N tile, "2sm" variants a CTA pair per 256 x TILE_N tile (tcgen05 cta_group::2); "_k512"
// selects 512-K pipeline stages (128-byte weight rows per TMA box) instead of 256-K stages.
struct Kind { const char* name; bool two_sm; int tile_n; int stage_k; };
const Kind kKinds[] = {
    {"sparse_2sm_256x128", true, 128, 256},     {"sparse_2sm_256x256", true, 256, 256},
    {"sparse_1sm_128x128", false, 128, 256},    {"sparse_1sm_128x256", false, 256, 256},
    {"sparse_2sm_256x64", true, 64, 256},       {"sparse_1sm_128x64", false, 64, 256},
    {"sparse_2sm_256x64_k512", true, 64, 512},  {"sparse_1sm_128x64_k512", false, 64, 512},
    {"sparse_1sm_128x128_k512", false, 128, 512},
};
constexpr int kNumKinds = sizeof(kKinds) / sizeof(kKinds[0]);

}  // namespace
}  // namespace pnv

using namespace pnv;

// Split-K workspace of the narrow kernel: one arrival counter per (expert, M tile), padded to 256 bytes, then two
// partial-accumulator slots of 128 x tile_n floats per CTA.
static long long split_counter_bytes(int experts, int features) {
  return ((long long)experts * ceil_div_i(features, kTileM) * 4 + 255) / 256 * 256;
}
static int narrow_tile_n(int max_n) { return max_n <= 16 ? 16 : 32; }

extern "C" int64_t pnv_group_mm_workspace_bytes(int experts, int features, int max_n, int sm_count) {
  if (experts < 1 || features < 1 || max_n < 1 || max_n > 32) return 0;   // wide tiles are never split
  if (sm_count <= 0) sm_count = 148;
  return split_counter_bytes(experts, features) + 2LL * sm_count * kTileM * narrow_tile_n(max_n) * 4;
}

extern "C" int pnv_group_mm_num_configs(void) { return kNumKinds; }

extern "C" const char* pnv_group_mm_config_name(int config_id) {
  return (config_id >= 0 && config_id < kNumKinds) ? kKinds[config_id].name : nullptr;
}

extern "C" int pnv_group_mm_device_status(int* status_out) {
  PNV_REQUIRE(status_out, "null pointer argument");
  PNV_CUDA(cudaDeviceSynchronize());
  PNV_CUDA(cudaMemcpyFromSymbol(status_out, g_status, sizeof(int)));
  int zero = 0;
  PNV_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(int)));
  return PNV_OK;
}

namespace pnv {
namespace {

// Self-test of the give-up path of the bounded waits: one thread waits, with a short poll budget, on a
// barrier that nothing ever arrives on.  No copy is in flight and no tensor memory is held, so giving
// up is all there is to do: record the code, invalidate the barrier, return.
__global__ void bounded_wait_probe_kernel(int* gave_up) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    ptx::fence_mbar_init();
    const bool done = ptx::mbar_wait_limited(&bar, 0, 2048);
    if (!done) atomicExch(&g_status, kSelfTestTimeout);
    *gave_up = done ? 0 : 1;
    ptx::mbar_inval(&bar);
  }
}

struct FusedArgs {
  uint8_t* b_out = nullptr;
  uint8_t* sfb_out = nullptr;
  const float* gscale = nullptr;
  int gpe = 0;
  GatedAct act{PNV_ACT_SILU, 1.f, -1.f, nullptr};
};

// The tile variants of the fused op, by the reference's names (csrc/sm100/tactics.cu:52-57).
struct FusedKind { const char* name; bool two_sm; int base_config; };
const FusedKind kFusedKinds[] = {
    {"fused_2sm_256x64_k512", true, 6}, {"fused_2sm_256x64", true, 4},
    {"fused_1sm_128x64", false, 5},     {"fused_2sm_256x128", true, 0},
    {"fused_1sm_128x128", false, 2},    {"fused_2sm_256x256", true, 1},
};
constexpr int kNumFusedKinds = sizeof(kFusedKinds) / sizeof(kFusedKinds[0]);

int group_mm_common(void* out, const int32_t* row_map, const RowParts* out_parts, const FusedArgs* fused, const uint8_t* a_comp, const uint8_t* e_meta,
                    const uint8_t* sfa, const uint8_t* b_act, const uint8_t* sfb, const float* alphas,
                    const int32_t* counts, int experts, int features, int k, int max_n, int config_id,
                    int cluster_m, int cluster_n, int sm_count, int pdl, void* workspace, int64_t workspace_bytes,
                    pnv_stream_t stream, const char* display_name) {
  PNV_REQUIRE((out || out_parts) && a_comp && e_meta && sfa && b_act && sfb && alphas && counts, "null pointer argument");
  PNV_REQUIRE(experts >= 1 && features >= 1 && max_n >= 1, "experts, features and max_n must be positive");
  PNV_REQUIRE(experts <= kMaxExperts, "group_mm supports at most %d experts per call, got %d", kMaxExperts,
              experts);
  PNV_REQUIRE(k > 0 && k % kSfBlock == 0, "K must be a multiple of %d, got %d", kSfBlock, k);
  PNV_REQUIRE(config_id >= 0 && config_id < kNumKinds, "config_id must be in [0, %d), got %d", kNumKinds,
              config_id);
  const Kind& kind = kKinds[config_id];
  const char* name = display_name ? display_name : kind.name;
  auto pow2_le4 = [](int x) { return x == 1 || x == 2 || x == 4; };
  PNV_REQUIRE(pow2_le4(cluster_m) && pow2_le4(cluster_n) && cluster_m * cluster_n <= 16,
              "%s: cluster dims must be powers of two <= 4 with product <= 16, got %dx%d", name,
              cluster_m, cluster_n);
  PNV_REQUIRE(!kind.two_sm || cluster_m % 2 == 0,
              "%s is a 2SM kernel and needs an even cluster_m, got %d", name, cluster_m);
  PNV_REQUIRE((reinterpret_cast<uintptr_t>(a_comp) | reinterpret_cast<uintptr_t>(b_act) |
               reinterpret_cast<uintptr_t>(e_meta) | reinterpret_cast<uintptr_t>(sfa) |
               reinterpret_cast<uintptr_t>(sfb) | reinterpret_cast<uintptr_t>(out)) % 16 == 0,
              "group_mm operands must be 16-byte aligned");
  if (sm_count <= 0) {
    int dev = 0;
    PNV_CUDA(cudaGetDevice(&dev));
    PNV_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }

  WeightDims wd = weight_dims(features, k);
  Params p;
  p.e_meta = e_meta; p.sfa = sfa; p.sfb = sfb; p.alphas = alphas; p.counts = counts;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.row_map = row_map;
  p.out_parts = out_parts ? *out_parts : RowParts{};
  p.f_b_out = nullptr; p.f_sfb_out = nullptr; p.f_gscale = nullptr; p.f_gpe = 0; p.f_n = 0; p.f_n_kt = 0;
  p.f_act = GatedAct{PNV_ACT_SILU, 1.f, -1.f, nullptr};
  if (fused != nullptr) {
    p.f_b_out = fused->b_out; p.f_sfb_out = fused->sfb_out; p.f_gscale = fused->gscale; p.f_gpe = fused->gpe;
    p.f_n = features / 2; p.f_n_kt = sf_k_atoms(features / 2); p.f_act = fused->act;
  }
  p.E = experts; p.M = features; p.K = k; p.max_n = max_n;
  p.n_mt = ceil_div_i(features, kTileM);
  p.n_kt = sf_k_atoms(k);
  p.e_k_atoms = wd.k_e / 16;
  p.e_m_atoms = wd.m_e / 128;
  p.sfb_rt = sf_row_atoms(max_n);
  p.stages = 0;
  p.prod_lanes = 1;
  p.b_tail = 0;
  p.split_counters = nullptr;
  p.split_partials = nullptr;

  // Tile geometry.  The variant names fix the widest token tile; when every expert's tokens fit one
  // narrow tile (max_n <= 32) the kernel runs 16- or 32-wide MMAs over 512-K stages with four issuer
  // warps instead: same results, far less padding and a deeper pipeline.
  int tile_n = kind.tile_n, stage_k = kind.stage_k;
  const bool narrow = max_n <= 32;
  if (narrow) {
    tile_n = max_n <= 16 ? 16 : 32;
    stage_k = 512;
  }
  const bool pair = kind.two_sm && !narrow;
  // The 256 x 256 pair kernel takes 512-K stages (three large ones instead of six) when K is long: every stage
  // costs the lone issuing threads the same few hundred cycles whatever it holds, and a long K loop keeps a short
  // ring busy (measured: K = 7168 -5 to -12 %, K = 3072 -10 %; K = 2048 +4 %, K = 768 +3 %).
  if (pair && tile_n == 256 && stage_k == 256 && k >= 3072) stage_k = 512;
  p.k_stages = ceil_div_i(k, stage_k);
  // the split schedule counts K stages in 32 bits
  const bool split_fits = (long long)experts * p.n_mt * p.k_stages < (1LL << 30);
  if (narrow && workspace != nullptr && p.k_stages > 1 && split_fits) {
    const int64_t need = pnv_group_mm_workspace_bytes(experts, features, max_n, sm_count);
    PNV_REQUIRE(workspace_bytes >= need, "group_mm: the split-K workspace holds %lld bytes, %lld are needed",
                (long long)workspace_bytes, (long long)need);
    PNV_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "group_mm: the workspace must be 256-byte aligned");
    p.split_counters = reinterpret_cast<int*>(workspace);
    p.split_partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + split_counter_bytes(experts, features));
  }

  CUtensorMap map_a, map_b, map_b_tail;
  if (int rc = make_map(&map_a, a_comp, (uint64_t)wd.k_ac / 2, (uint64_t)wd.m_ac, (uint64_t)experts,
                        (uint32_t)stage_k / 4, (uint32_t)kTileM,
                        stage_k == 512 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B))
    return rc;
  // token rows per activation copy: a CTA of a pair loads half of the tile
  const uint32_t box_rows = (uint32_t)(pair ? tile_n / 2 : tile_n);
  p.b_4d = k % 256 == 0 ? 1 : 0;
  if (p.b_4d) {
    if (int rc = make_map_b4(&map_b, b_act, (uint64_t)k / 2, (uint64_t)max_n, (uint64_t)experts, box_rows,
                             (uint32_t)stage_k / 256))
      return rc;
  } else if (int rc = make_map(&map_b, b_act, (uint64_t)k / 2, (uint64_t)max_n, (uint64_t)experts, 128, box_rows,
                               CU_TENSOR_MAP_SWIZZLE_128B)) {
    return rc;
  }
  // narrow tail tiles: tiles of 128 tokens or more, activations through the 4-D map
  map_b_tail = map_b;
#ifndef PNV_NO_TAIL_TILES      // developer builds: every tile at full width, for comparisons
  if (!narrow && tile_n >= 128 && p.b_4d) {
    if (int rc = make_map_b4(&map_b_tail, b_act, (uint64_t)k / 2, (uint64_t)max_n, (uint64_t)experts,
                             (uint32_t)(pair ? 32 : 64), (uint32_t)stage_k / 256))
      return rc;
    p.b_tail = 1;
  }
#endif

  cudaStream_t s = (cudaStream_t)stream;
  const bool use_pdl = pdl != 0 && pdl_enabled();
  if (narrow) {
    if (tile_n == 16) return launch_narrow<16, 512, 4>(map_a, map_b, p, sm_count, use_pdl, s);
    return launch_narrow<32, 512, 4>(map_a, map_b, p, sm_count, use_pdl, s);
  }
  switch (tile_n * 1000 + stage_k + (pair ? 1 : 0)) {
    case 64256: return launch_wide<64, 256, false>(map_a, map_b, map_b_tail, p, sm_count, use_pdl, s);
    case 64257: return launch_wide<64, 256, true>(map_a, map_b, map_b_tail, p, sm_count, use_pdl, s);
    case 64512: return launch_wide<64, 512, false>(map_a, map_b, map_b_tail, p, sm_count, use_pdl, s);
    case 64513: return launch_wide<64, 512, true>(map_a, map_b, map_b_tail, p, sm_count, use_pdl, s);
    case 128256: return launch_wide<128, 256, false>(map_a, map_b, map_b_tail, p, sm_count, use_pdl, s);
    case 128257: return launch_wide<128, 256, true>(map_a, map_b, map_b_tail, p, sm_count, use_pdl, s);
    case 128512: return launch_wide<128, 512, false>(map_a, map_b, map_b_tail, p, sm_count, use_pdl, s);
    case 256256: return launch_wide<256, 256, false>(map_a, map_b, map_b_tail, p, sm_count, use_pdl, s);
    case 256257: return launch_wide<256, 256, true>(map_a, map_b, map_b_tail, p, sm_count, use_pdl, s);
    case 256513: return launch_wide<256, 512, true>(map_a, map_b, map_b_tail, p, sm_count, use_pdl, s);
    default: break;
  }
  return fail(PNV_ERR_UNSUPPORTED, "group_mm: no kernel for tile %dx%d%s", tile_n, stage_k, pair ? " (pair)" : "");
}

}  // namespace
}  // namespace pnv

#ifdef PNV_WIDE_PROFILE
// developer build only: read and clear the wide kernel's cycle counters (16 per CTA, 296 CTAs)
extern "C" int pnv_debug_wide_profile(long long* out) {
  PNV_CUDA(cudaDeviceSynchronize());
  PNV_CUDA(cudaMemcpyFromSymbol(out, g_wide_prof, sizeof(long long) * 296 * 16));
  static long long zeros[296 * 16] = {};
  PNV_CUDA(cudaMemcpyToSymbol(g_wide_prof, zeros, sizeof(zeros)));
  return PNV_OK;
}
#endif

extern "C" int pnv_selftest_bounded_wait(int* gave_up_out) {
  PNV_REQUIRE(gave_up_out, "null pointer argument");
  int* flag = nullptr;
  PNV_CUDA(cudaMalloc(reinterpret_cast<void**>(&flag), sizeof(int)));
  bounded_wait_probe_kernel<<<1, 32>>>(flag);
  cudaError_t err = cudaGetLastError();
  if (err == cudaSuccess) err = cudaMemcpy(gave_up_out, flag, sizeof(int), cudaMemcpyDeviceToHost);
  cudaFree(flag);
  if (err != cudaSuccess) return fail(PNV_ERR_CUDA, "bounded-wait self-test failed: %s", cudaGetErrorString(err));
  return PNV_OK;
}

extern "C" int pnv_group_mm(void* out, const uint8_t* a_comp, const uint8_t* e_meta, const uint8_t* sfa,
                            const uint8_t* b_act, const uint8_t* sfb, const float* alphas,
                            const int32_t* counts, int experts, int features, int k, int max_n,
                            int config_id, int cluster_m, int cluster_n, int sm_count, int pdl,
                            void* workspace, int64_t workspace_bytes, pnv_stream_t stream) {
  return group_mm_common(out, nullptr, nullptr, nullptr, a_comp, e_meta, sfa, b_act, sfb, alphas, counts, experts, features, k,
                         max_n, config_id, cluster_m, cluster_n, sm_count, pdl, workspace, workspace_bytes, stream,
                         nullptr);
}

extern "C" int pnv_group_mm_rows(void* out, const int32_t* row_map, const uint8_t* a_comp, const uint8_t* e_meta,
                                 const uint8_t* sfa, const uint8_t* b_act, const uint8_t* sfb, const float* alphas,
                                 const int32_t* counts, int experts, int features, int k, int max_n, int config_id,
                                 int cluster_m, int cluster_n, int sm_count, int pdl, void* workspace,
                                 int64_t workspace_bytes, pnv_stream_t stream) {
  PNV_REQUIRE(row_map, "null pointer argument");
  return group_mm_common(out, row_map, nullptr, nullptr, a_comp, e_meta, sfa, b_act, sfb, alphas, counts, experts, features, k,
                         max_n, config_id, cluster_m, cluster_n, sm_count, pdl, workspace, workspace_bytes, stream,
                         nullptr);
}

extern "C" int pnv_group_mm_rows_parts(void* const* out_parts, int n_parts, int64_t rows_per_part, const int32_t* row_map,
                                       const uint8_t* a_comp, const uint8_t* e_meta, const uint8_t* sfa,
                                       const uint8_t* b_act, const uint8_t* sfb, const float* alphas,
                                       const int32_t* counts, int experts, int features, int k, int max_n, int config_id,
                                       int cluster_m, int cluster_n, int sm_count, int pdl, void* workspace,
                                       int64_t workspace_bytes, pnv_stream_t stream) {
  PNV_REQUIRE(row_map, "null pointer argument");
  RowParts parts;
  if (int rc = make_row_parts(out_parts, n_parts, rows_per_part, parts)) return rc;
  return group_mm_common(nullptr, row_map, &parts, nullptr, a_comp, e_meta, sfa, b_act, sfb, alphas, counts, experts,
                         features, k, max_n, config_id, cluster_m, cluster_n, sm_count, pdl, workspace, workspace_bytes,
                         stream, nullptr);
}

extern "C" int pnv_group_mm_swiglu_num_configs(void) { return kNumFusedKinds; }

extern "C" const char* pnv_group_mm_swiglu_config_name(int config_id) {
  return (config_id >= 0 && config_id < kNumFusedKinds) ? kFusedKinds[config_id].name : nullptr;
}

extern "C" int pnv_group_mm_swiglu_quant(uint8_t* b_out, uint8_t* sfb_out, const uint8_t* a_comp,
                                         const uint8_t* e_meta, const uint8_t* sfa, const uint8_t* b_act,
                                         const uint8_t* sfb, const float* alphas, const int32_t* counts,
                                         const float* gscale, int gscale_per_expert, int experts,
                                         int features, int k, int max_n, int config_id, int cluster_m,
                                         int cluster_n, int act_kind, float beta, float linear_beta,
                                         int sm_count, int pdl, void* workspace, int64_t workspace_bytes,
                                         pnv_stream_t stream) {
  PNV_REQUIRE(b_out && sfb_out && gscale, "null pointer argument");
  PNV_REQUIRE(features % 128 == 0,
              "features (2N) must be a multiple of 128 (whole 64-row gate/up blocks per CTA), got %d", features);
  PNV_REQUIRE(config_id >= 0 && config_id < kNumFusedKinds, "config_id must be in [0, %d), got %d",
              kNumFusedKinds, config_id);
  PNV_REQUIRE((reinterpret_cast<uintptr_t>(b_out) | reinterpret_cast<uintptr_t>(sfb_out)) % 16 == 0,
              "group_mm operands must be 16-byte aligned");
  FusedArgs f;
  if (int rc = make_gated_act(act_kind, beta, linear_beta, (cudaStream_t)stream, f.act)) return rc;
  f.b_out = b_out; f.sfb_out = sfb_out; f.gscale = gscale; f.gpe = gscale_per_expert ? 1 : 0;
  PNV_REQUIRE(experts >= 1 && max_n >= 1, "experts and max_n must be positive");
  PNV_REQUIRE(sf_numel(max_n, features / 2, experts) < (1LL << 31), "sfb_out must be smaller than 2 GiB");
  const FusedKind& fk = kFusedKinds[config_id];
  return group_mm_common(b_out, nullptr, nullptr, &f, a_comp, e_meta, sfa, b_act, sfb, alphas, counts, experts, features, k, max_n,
                         fk.base_config, cluster_m, cluster_n, sm_count, pdl, workspace, workspace_bytes, stream, fk.name);
}
