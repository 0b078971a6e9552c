// group_mm: out[e, t, :] = bf16(alpha[e] * W[e] * x[e, t, :]) for t < counts[e], with W stored
// paired-4:8 sparse NVFP4 (a_comp + e_meta + sfa) and x stored NVFP4 (b_act + sfb).
//
// Two persistent kernels, one CTA per SM.  group_mm_kernel (this comment) runs the narrow token
// tiles of decode-sized problems; group_mm_wide_kernel (further down) the 64- to 256-wide tiles.
// Narrow kernel, four warp roles (6 + ISSUERS warps):
//   warp 0 (one lane)  tile producer: per K stage, the TMA tile loads of the compressed weights and
//                      of the activations (one 3-D tensor map each covers every expert; 128-byte
//                      swizzle, or 64-byte swizzle for the weights of a 256-K stage);
//   warp 1 (one lane)  side producer: plain bulk copies of the metadata atoms and of the SFA / SFB
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
#include <cstdlib>
#include <mutex>

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
  kSideProducerTimeout = 5, kMmaScaleTimeout = 6, kScaleLoaderTimeout = 7
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
  int b_res_bytes;   // wide kernel: bytes of the resident activation tile in front of the stage ring (0 = streamed)
  // fused SwiGLU + requantise epilogue (kFused kernels): GEMM2's operands instead of a bf16 output
  uint8_t* f_b_out;        // [E, max_n, N/2] e2m1 codes, N = M / 2
  uint8_t* f_sfb_out;      // swizzled scales for (max_n, N), pre-filled with 0x38
  const float* f_gscale;   // GEMM2 activation global scale, [E] or [1]
  int f_gpe;
  int f_n;                 // N
  int f_n_kt;              // scale K-atoms of the N-wide output
  GatedAct f_act;
  long long* prof;   // optional per-CTA cycle counters (8 per CTA): see PNV_GROUP_MM_PROFILE
  unsigned* trace;   // traced build only: host-mapped breadcrumb words, 16 per CTA (first 8 CTAs)
};

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

// Traced build (kTrace): every asynchronous operation is issued alone and waited for, each step
// leaves a breadcrumb in host-mapped memory (readable even after a fault killed the context), and
// every copy's addresses and size are checked first; a failed check is recorded and the copy is
// skipped.  Breadcrumb slots per CTA: 0 setup, 1 tile producer, 2 MMA issuer, 3 epilogue,
// 4 first failed check (code) with its operands in 5..7, 11 side producer.
template <bool kTrace>
__device__ __forceinline__ void crumb(unsigned* trace, int slot, unsigned code) {
  if (kTrace && trace != nullptr && blockIdx.x < 8) {
    volatile unsigned* t = trace + blockIdx.x * 16 + slot;
    *t = code;
    __threadfence_system();
  }
}
template <bool kTrace>
__device__ __forceinline__ bool check_copy(unsigned* trace, unsigned code, uint32_t dst, uint64_t src,
                                           uint32_t bytes, uint32_t dst_align) {
  if (!kTrace) return true;
  if ((dst % dst_align) == 0 && (src % 16) == 0 && (bytes % 16) == 0) return true;
  if (trace != nullptr && blockIdx.x < 8) {
    volatile unsigned* t = trace + blockIdx.x * 16;
    if (t[4] == 0) { t[4] = code; t[5] = dst; t[6] = (unsigned)(src & 0xFFFFFFFFu); t[7] = bytes; }
    __threadfence_system();
  }
  return false;
}

__device__ __forceinline__ void epilogue_bar_sync() {
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

template <int TILE_N, int STAGE_K, int ISSUERS, bool kTrace, bool kFused>
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
  uint64_t* dbg_bar = acc_empty + C::kAccStages;     // 2 + ISSUERS extra barriers, used by the traced build
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dbg_bar + 2 + ISSUERS);
  int* s_counts = reinterpret_cast<int*>(smem + C::kStages * C::kStageBytes + kOutStageBytes + 256);
#define CRUMB(slot, code) crumb<kTrace>(p.trace, slot, code)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- setup that does not depend on the previous kernel ---------------------------------------
  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    // arrivals on a stage's full barrier: the tile producer and the two bulk-copy lanes (one in the traced build)
    for (int s = 0; s < C::kStages; ++s) { ptx::mbar_init(full_bar + s, kTrace ? 2 : 3); ptx::mbar_init(empty_bar + s, ISSUERS); }
    for (int a = 0; a < C::kAccStages; ++a) {
      ptx::mbar_init(acc_full + a, ISSUERS);
      ptx::mbar_init(acc_empty + a, kEpilogueThreads);
    }
    for (int d = 0; d < 2 + ISSUERS; ++d) ptx::mbar_init(dbg_bar + d, 1);
    ptx::fence_mbar_init();
    CRUMB(0, 1);
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
  if (threadIdx.x == 0) { CRUMB(0, 3); CRUMB(8, tmem_base); CRUMB(9, ptx::smem_u32(smem)); }

  TileWalk walk;
  walk.init<TILE_N>(s_counts, p.E, p.n_mt);

  if (warp == 0) {
    // =============================== tile producer (TMA) ===============================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, dphase = 0;
      (void)dphase;
      bool ok = true;
      for (long long t = blockIdx.x; ok; t += gridDim.x) {
        int mt, nt;
        if (!walk.seek<TILE_N>(t, mt, nt)) break;
        const int e = walk.e;
        const int n0 = nt * TILE_N;
#pragma unroll 1
        for (int ks = 0; ks < p.k_stages; ++ks) {
          long long tq0 = p.prof ? clock64() : 0;
          if (!ptx::mbar_wait(empty_bar + stage, phase ^ 1)) {
            atomicExch(&g_status, kProducerEmptyTimeout);
            ok = false;
            break;
          }
          if (p.prof) p.prof[blockIdx.x * 8 + 4] += clock64() - tq0;
          uint8_t* st = stage_base + stage * C::kStageBytes;
          const int k_atoms = min(C::kAtoms, p.n_kt - ks * C::kAtoms);
          const int b_boxes = (k_atoms + 1) / 2;
          if (!kTrace) {
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
          } else {
            auto one = [&](unsigned code, uint32_t bytes, auto issue) {
              CRUMB(1, code);
              ptx::mbar_arrive_expect_tx(dbg_bar, bytes);
              issue();
              bool done = ptx::mbar_wait(dbg_bar, dphase);
              dphase ^= 1;
              CRUMB(1, code + (done ? 1 : 2));
            };
            if (check_copy<kTrace>(p.trace, 100, ptx::smem_u32(st + C::kOffA), 0, C::kABytes, 1024))
              one(110, C::kABytes, [&] {
                ptx::tma_load_3d(st + C::kOffA, &map_a, dbg_bar, ks * C::kARowBytes, mt * kTileM, e);
              });
            for (int b = 0; b < b_boxes; ++b)
              if (check_copy<kTrace>(p.trace, 101, ptx::smem_u32(st + C::kOffB + b * C::kBBoxBytes), 0,
                                     C::kBBoxBytes, 1024))
                one(120, C::kBBoxBytes, [&] {
                  ptx::tma_load_3d(st + C::kOffB + b * C::kBBoxBytes, &map_b, dbg_bar,
                                   ks * (STAGE_K / 2) + b * 128, n0, e);
                });
            ptx::mbar_arrive(full_bar + stage);
            CRUMB(1, 160);
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
    // expect-tx arrival; the traced build keeps everything in lane 0
    if (lane < (kTrace ? 1 : 2)) {
      int stage = 0;
      uint32_t phase = 0, dphase = 0;
      (void)dphase;
      bool ok = true;
      for (long long t = blockIdx.x; ok; t += gridDim.x) {
        int mt, nt;
        if (!walk.seek<TILE_N>(t, mt, nt)) break;
        const int e = walk.e;
        const int n0 = nt * TILE_N;
        const uint8_t* e_base = p.e_meta + (((long long)e * p.e_k_atoms) * p.e_m_atoms + mt) * 2048;
        const uint8_t* sfa_base = p.sfa + (((long long)e * p.n_mt + mt) * p.n_kt) * 512;
        const uint8_t* sfb_base = p.sfb + (((long long)e * p.sfb_rt + (n0 >> 7)) * p.n_kt) * 512;
        const int sfb_row_atoms = TILE_N > 128 ? min(2, p.sfb_rt - (n0 >> 7)) : 1;
        for (int ks = 0; ks < p.k_stages; ++ks) {
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
          if (!kTrace) {
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
          } else {
            auto one = [&](unsigned code, uint32_t bytes, auto issue) {
              CRUMB(11, code);
              ptx::mbar_arrive_expect_tx(dbg_bar + 1, bytes);
              issue();
              bool done = ptx::mbar_wait(dbg_bar + 1, dphase);
              dphase ^= 1;
              CRUMB(11, code + (done ? 1 : 2));
            };
            for (int ea = 0; ea < e_atoms; ++ea) {
              const uint8_t* src = e_base + (long long)(ks * C::kEAtoms + ea) * p.e_m_atoms * 2048;
              if (check_copy<kTrace>(p.trace, 102, ptx::smem_u32(st + C::kOffE + ea * 2048), (uint64_t)src, 2048, 16))
                one(130, 2048, [&] { ptx::bulk_load(st + C::kOffE + ea * 2048, src, 2048, dbg_bar + 1); });
            }
            if (check_copy<kTrace>(p.trace, 103, ptx::smem_u32(st + C::kOffSfa), (uint64_t)sfa_src, sf_bytes, 16))
              one(140, sf_bytes, [&] { ptx::bulk_load(st + C::kOffSfa, sfa_src, sf_bytes, dbg_bar + 1); });
            for (int ra = 0; ra < sfb_row_atoms; ++ra) {
              const uint8_t* src = sfb_base + ((long long)ra * p.n_kt + ks * C::kAtoms) * 512;
              if (check_copy<kTrace>(p.trace, 104, ptx::smem_u32(st + C::kOffSfb + ra * C::kSfaBytes),
                                     (uint64_t)src, sf_bytes, 16))
                one(150, sf_bytes, [&] {
                  ptx::bulk_load(st + C::kOffSfb + ra * C::kSfaBytes, src, sf_bytes, dbg_bar + 1);
                });
            }
            ptx::mbar_arrive(full_bar + stage);
            CRUMB(11, 160);
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
      uint32_t phase = 0, acc_phase = 0, dphase = 0;
      (void)dphase;
      bool ok = true;
      long long c_wait_full = 0, c_issue = 0, c_wait_acc = 0, n_stage = 0;
      const bool prof = p.prof != nullptr && issuer == 0;
      for (long long t = blockIdx.x; ok; t += gridDim.x) {
        int mt, nt;
        if (!walk.seek<TILE_N>(t, mt, nt)) break;
        long long tp0 = prof ? clock64() : 0;
        if (!ptx::mbar_wait(acc_empty + acc, acc_phase ^ 1)) {
          atomicExch(&g_status, kMmaAccTimeout);
          break;
        }
        ptx::tc_fence_after();
        if (prof) c_wait_acc += clock64() - tp0;
        const uint32_t d_tmem = tmem_base + (acc * ISSUERS + issuer) * TILE_N;
        // The scales of a 64-wide tile's rows sit 0 or 2 columns into the 128-row atom.  The MMA
        // faults (misaligned address) on an odd column offset, which is why 16- and 32-wide tiles
        // exist only for problems with a single token tile (offset 0).
        const uint32_t sfb_col = tmem_base + kColSfb + (TILE_N < 128 ? ((nt * TILE_N) & 127) >> 5 : 0);
        for (int ks = 0; ks < p.k_stages; ++ks) {
          long long tp1 = prof ? clock64() : 0;
          if (!ptx::mbar_wait(full_bar + stage, phase)) {
            atomicExch(&g_status, kMmaFullTimeout);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          long long tp2 = prof ? clock64() : 0;
          if (prof) { c_wait_full += tp2 - tp1; ++n_stage; }
          const uint32_t st = ptx::smem_u32(stage_base + stage * C::kStageBytes);
          const int k_atoms = min(C::kAtoms, p.n_kt - ks * C::kAtoms);
          auto settle = [&](unsigned code) {   // traced build: wait until the operation just issued retires
            if (kTrace) {
              CRUMB(2, code);
              ptx::tc_commit(dbg_bar + 2 + issuer);
              bool done = ptx::mbar_wait(dbg_bar + 2 + issuer, dphase);
              dphase ^= 1;
              CRUMB(2, code + (done ? 1 : 2));
            }
          };
          if (ka0 < k_atoms) {
            // metadata atoms covering this issuer's K-blocks, into its private columns
#pragma unroll
            for (int i = 0; i < C::kEAtomsPerIssuer; ++i) {
              const int ea = ka0 / 2 + i;
              if (2 * ea < k_atoms)
                ptx::tc_cp_128x128b(e_cols + i * 4, ptx::smem_desc(st + C::kOffE + ea * 2048, 128, 0, 0));
            }
          }
          settle(210);
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
          settle(220);
#pragma unroll
          for (int i = 0; i < kPer; ++i) {
            const int ka = ka0 + i;
            if (ka < k_atoms) {
              const uint64_t a_desc = ptx::smem_desc(st + C::kOffA + ka * 32, 8 * C::kARowBytes, 16, C::kASwizzle);
              const uint64_t b_desc =
                  ptx::smem_desc(st + C::kOffB + (ka >> 1) * C::kBBoxBytes + (ka & 1) * 64, 1024, 16, 2);
              // metadata columns: 2 per K-block inside the atom that holds it
              const uint32_t e_tmem = e_cols + (kPer >= 2 ? i * 2 : (ka & 1) * 2);
              ptx::tc_mma_sp_nvf4(d_tmem, a_desc, b_desc, idesc, (ks | i) != 0 ? 1u : 0u,
                                  tmem_base + kColSfa + ka * 4, sfb_col + ka * C::kSfbColsPerAtom, e_tmem);
              settle(240 + 10 * i);
            }
          }
          ptx::tc_commit(empty_bar + stage);   // stage reusable once every issuer's MMAs and copies retire
          if (prof) c_issue += clock64() - tp2;
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        ptx::tc_commit(acc_full + acc);        // this issuer's partial accumulator is complete
        if (kTrace) CRUMB(2, 290);
        if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
      }
      if (prof) {
        long long* q = p.prof + blockIdx.x * 8;
        q[0] = c_wait_full; q[1] = c_issue; q[2] = c_wait_acc; q[3] = n_stage;
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
    for (long long t = blockIdx.x;; t += gridDim.x) {
      int mt, nt;
      if (!walk.seek<TILE_N>(t, mt, nt)) break;
      const int e = walk.e;
      const int cnt = s_counts[e];
      const bool eprof = p.prof != nullptr && ep_tid == 0;
      long long te0 = eprof ? clock64() : 0;
      if (!ptx::mbar_wait(acc_full + acc, acc_phase)) {
        atomicExch(&g_status, kEpilogueTimeout);
        break;
      }
      ptx::tc_fence_after();
      long long te1 = eprof ? clock64() : 0;
      long long t_ld = 0;
      if (kTrace && ep_tid == 0) CRUMB(3, 300);
      const float alpha = p.alphas[e];
      const int n0 = nt * TILE_N;
      __nv_bfloat16* out_e = p.out + (long long)e * p.max_n * p.M;
      // issuers whose K-blocks exist for this K (a short K leaves the later issuers idle)
      const int live = min(ISSUERS, ceil_div_i(min(C::kAtoms, p.n_kt), C::kAtomsPerIssuer));
#pragma unroll 1
      for (int c0 = 0; c0 < TILE_N; c0 += 32) {
        if (n0 + c0 >= cnt) break;             // uniform over the four epilogue warps
        uint32_t r[32];
        const uint32_t lane_base = tmem_base + ((uint32_t)(sub * 32) << 16) + c0;
        long long tl0 = eprof ? clock64() : 0;
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
        if (eprof) t_ld += clock64() - tl0;
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
            if (n < cnt && m < p.M)
              *reinterpret_cast<uint4*>(out_e + (long long)n * p.M + m) =
                  *reinterpret_cast<const uint4*>(buf + row * kOutRow + col);
          }
          ++chunk;
        } else {
          const int m = mt * kTileM + m_local;
          if (m < p.M) {
#pragma unroll
            for (int i = 0; i < (TILE_N < 32 ? TILE_N : 32); ++i) {
              const int n = n0 + c0 + i;
              if (n < cnt)
                out_e[(long long)n * p.M + m] = __float2bfloat16_rn(__fmul_rn(alpha, __uint_as_float(r[i])));
            }
          }
        }
      }
      if (kTrace && ep_tid == 0) CRUMB(3, 320);
      ptx::tc_fence_before();
      ptx::mbar_arrive(acc_empty + acc);
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
      if (eprof) {   // waiting for an accumulator, reading it, the rest of the tile's epilogue
        long long* q = p.prof + blockIdx.x * 8;
        if (!kFused) { q[5] += te1 - te0; q[6] += t_ld; } q[7] += clock64() - te1 - t_ld;
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
    if (lane == 0) CRUMB(0, 9);
  }
#undef CRUMB
}

// ---- wide tiles (TILE_N >= 64) ---------------------------------------------------------------------
//
// With 64- to 256-wide token tiles the narrow kernel's single issuer thread is the bottleneck: per
// 128-K block it issues one MMA but also two or three tcgen05.cp of scale atoms, and every
// tcgen05 operation costs the issuing thread 50-100 cycles.  This kernel takes the scales off that
// thread.  Sixteen warps:
//   warp 0   tile producer (TMA: compressed weights, activations)        } as in the narrow kernel
//   warp 1   side producer (bulk copies: metadata, SFA, SFB atoms)       }
//   2 - 3    MMA issuers, alternate tiles: per stage the metadata tcgen05.cp and the MMAs, nothing else
//   4 - 7    scale loaders, one per tensor-memory lane quarter: read the stage's scale atoms from
//            shared memory (one 16-byte line per lane) and write them into a ring of scale slots in
//            tensor memory with tcgen05.st -- the same image tcgen05.cp.32x128b.warpx4 would leave
//   8 - 15   epilogue, two groups of four warps; a tile's 32-column chunks alternate between them
// Every pipeline stage owns one slot of the scale ring.  Barriers: full[s] (copies landed; the
// loaders wait on it), sf_full[s] (the four loaders -> issuer: scales are in tensor memory, which
// also tells the issuer that the stage's copies have landed, since the loaders saw full[s] first),
// empty[s] (issuer's tcgen05.commit plus the four loaders -> producers).  A refilled stage implies
// that the MMAs which read the slot's previous scales have retired, so the loaders need no barrier
// of their own for the slot.  The issuer thread is the kernel's critical resource -- one thread
// executes a few hundred instructions per microsecond at best -- so it does no tile arithmetic:
// it counts this CTA's tiles once and then only waits, issues and commits.
//
// Resident activations (kBRes).  An SM takes in about 48 bytes per cycle from L2, while one MMA reads
// 12 KB (N = 128) of operands from shared memory in 96 cycles, so a kernel that streams both
// operands through the stage ring runs at the fill rate, not the tensor rate.  When a whole
// activation tile (TILE_N tokens x K) fits beside the ring, the CTA's unit of work becomes
// (expert, token tile): the activation tile is loaded once, in 256-K chunks with a full/empty
// barrier pair each, and every weight tile of the expert streams against it.  The next unit's
// chunks are loaded while the last weight tile of this unit is still being multiplied.
template <int TILE_N, int STAGE_K, bool kBRes>
struct WideCfg {
  static_assert(TILE_N == 64 || TILE_N == 128 || TILE_N == 256, "wide tile widths: 64, 128, 256");
  static_assert(STAGE_K == 256 || STAGE_K == 512, "stage depths: 256, 512");
  static constexpr int kThreads = 512;
  static constexpr int kAtoms = STAGE_K / 128;
  static constexpr int kARowBytes = STAGE_K / 4;
  static constexpr int kABytes = kTileM * kARowBytes;
  static constexpr uint32_t kASwizzle = STAGE_K == 512 ? 2 : 4;
  static constexpr int kBBoxes = STAGE_K / 256;
  static constexpr int kBBoxBytes = TILE_N * 128;
  static constexpr int kBBytes = kBRes ? 0 : kBBoxes * kBBoxBytes;   // activation bytes inside a stage
  static constexpr int kEAtoms = STAGE_K / 256;
  static constexpr int kEBytes = 2048 * kEAtoms;
  static constexpr int kSfaBytes = 512 * kAtoms;
  static constexpr int kSfbRowAtoms = TILE_N > 128 ? 2 : 1;
  static constexpr int kSfbBytes = kSfaBytes * kSfbRowAtoms;
  static constexpr int kStageBytes = kABytes + kBBytes + kEBytes + kSfaBytes + kSfbBytes;
  static constexpr int kOutBytes = 2 * kOutStageBytes;     // fused epilogue: one double-buffered transpose tile per group
  static constexpr int kPlainOutBytes = 8 * 2 * 16 * 40 * 2;   // plain epilogue: two [16][40] bf16 pieces per warp
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kMaxStages = 12;
  static constexpr int kMaxChunks = 16;                     // resident activation tile: at most 16 x 256 K
  static constexpr int kAccStages = TILE_N == 256 ? 1 : 2;
  static constexpr int kColE = 256;                         // tensor-memory columns: accumulators below 256
  static constexpr int kColSf = 272;                        // ring of scale slots
  static constexpr int kSfbColsPerAtom = 4 * kSfbRowAtoms;
  static constexpr int kSfSlotCols = kAtoms * (4 + kSfbColsPerAtom);
  static constexpr int kSfSlots = (kTmemCols - kColSf) / kSfSlotCols;   // one per stage: caps the pipeline depth
  static constexpr int kOffA = 0;
  static constexpr int kOffB = kABytes;
  static constexpr int kOffE = kOffB + kBBytes;
  static constexpr int kOffSfa = kOffE + kEBytes;
  static constexpr int kOffSfb = kOffSfa + kSfaBytes;
  static_assert(kStageBytes % 1024 == 0, "stage buffers must keep 1024-byte alignment");
  static_assert(kAccStages * TILE_N <= kColE && kColE + 2 * 4 * kEAtoms <= kColSf && kSfSlots >= 2,
                "tensor-memory column map overflows");
  static_assert(8 * (3 * kMaxStages + 2 * kAccStages + 2 * kMaxChunks) + 16 <= kBarrierBytes, "barrier block overflows");
};

// Barrier of one gate/up warp pair of the fused epilogue (lane quarters 0-1 or 2-3 of a group): the pair owns
// one 64-row block of the tile (32 gate rows, the 32 matching up rows) and shares nothing with the other pair.
__device__ __forceinline__ void epilogue_pair_sync(int group, int sub) {
  asm volatile("bar.sync %0, 64;" ::"r"(1 + group * 2 + (sub >> 1)) : "memory");
}

__device__ __forceinline__ uint64_t pack_desc(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Work items (tiles, or (expert, token tile) units when per_expert == 1) this CTA will process:
// items b, b + grid, ... of the list every role walks.  Warp-collective.
template <int TILE_N>
__device__ __forceinline__ int my_work_items(const int* cnt, int E, int per_expert, int lane) {
  long long sum = 0;
  for (int e = lane; e < E; e += 32) sum += ceil_div_i(cnt[e], TILE_N);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const long long total = sum * per_expert;
  return (long long)blockIdx.x < total ? (int)((total - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
}

// One work item of a CTA: a single tile, or with resident activations every weight tile of one
// (expert, token tile).  Returns false when the list is exhausted.
template <int TILE_N, bool kBRes>
__device__ __forceinline__ bool next_work(TileWalk& walk, long long w, int n_mt, int& mt_lo, int& mt_hi, int& nt) {
  int mt;
  if (!walk.seek<TILE_N>(w, mt, nt)) return false;
  if (kBRes) { mt_lo = 0; mt_hi = n_mt; } else { mt_lo = mt; mt_hi = mt + 1; }
  return true;
}

template <int TILE_N, int STAGE_K, bool kFused, bool kBRes>
__global__ void __launch_bounds__(512, 1)
group_mm_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const Params p) {
  using C = WideCfg<TILE_N, STAGE_K, kBRes>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* b_res = smem;                                   // resident activation tile (kBRes), p.b_res_bytes
  uint8_t* stage_base = smem + p.b_res_bytes;
  uint8_t* after_stages = stage_base + p.stages * C::kStageBytes;
  constexpr int kOutBytes = kFused ? C::kOutBytes : C::kPlainOutBytes;
  __nv_bfloat16* s_out = reinterpret_cast<__nv_bfloat16*>(after_stages);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(after_stages + kOutBytes);
  uint64_t* empty_bar = full_bar + C::kMaxStages;
  uint64_t* acc_full = empty_bar + C::kMaxStages;
  uint64_t* acc_empty = acc_full + C::kAccStages;
  uint64_t* sf_full = acc_empty + C::kAccStages;
  uint64_t* b_full = sf_full + C::kMaxStages;
  uint64_t* b_empty = b_full + C::kMaxChunks;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(b_empty + C::kMaxChunks);
  int* s_counts = reinterpret_cast<int*>(after_stages + kOutBytes + C::kBarrierBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(full_bar + s, 3);
      ptx::mbar_init(empty_bar + s, 1 + 4);
      ptx::mbar_init(sf_full + s, 4);
    }
    if (kBRes)
      for (int c = 0; c < C::kMaxChunks; ++c) { ptx::mbar_init(b_full + c, 1); ptx::mbar_init(b_empty + c, 1); }
    for (int a = 0; a < C::kAccStages; ++a) { ptx::mbar_init(acc_full + a, 1); ptx::mbar_init(acc_empty + a, 8); }
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  // counts (and everything else the producer kernels wrote) may only be read after this point
  pdl_wait();
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < p.E; i += C::kThreads) s_counts[i] = max(0, min(p.counts[i], p.max_n));
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  TileWalk walk;
  walk.init<TILE_N>(s_counts, p.E, kBRes ? 1 : p.n_mt);

  if (warp < 2) {
    // =============================== producers ===============================
    // warp 0: TMA tile copies (compressed weights, activations); warp 1: bulk copies of the
    // metadata, SFA and SFB atoms.  In each, p.prod_lanes lanes work side by side, lane i on
    // pipeline slots i, i + lanes, ...: one thread needs several hundred cycles per (wait, expect,
    // copy) sequence, while the same sequence issued by several lanes of a warp in one go costs
    // little more than once.  The loop carries its position (tile, K stage, slot, turn) forward with
    // additions only, and recomputes addresses only when the tile changes: a lone thread retires an
    // instruction every 6-20 cycles, so divisions per stage would cost as much as the copies.
    // The bulk-copy warp splits every stage between two lanes (metadata atoms; scale atoms), each with
    // its own expect-tx arrival, so a stage's full barrier counts three arrivals.
    const bool tile_role = warp == 0;
    const int slot_lane = tile_role ? lane : lane >> 1;     // which of the side-by-side pipeline slots
    const int part = lane & 1;                              // bulk-copy warp: 0 metadata, 1 scales
    if (slot_lane < p.prod_lanes) {
      bool ok = true;
      int n = 0, ks = slot_lane, stage = slot_lane, cur_n = -1;     // prod_lanes <= stages (host)
      uint32_t turn = 0;
      int e = 0, mt = 0, n0 = 0, sfb_row_atoms = 1;
      uint32_t uphase = 0;
      const uint8_t *e_base = nullptr, *sfa_base = nullptr, *sfb_base = nullptr;
      while (ok) {
        while (ks >= p.k_stages) { ks -= p.k_stages; ++n; }
        if (n != cur_n) {                                  // a new tile: where it is, and its operand bases
          int nt;
          if (kBRes) {
            const int u = n / p.n_mt;
            mt = n - u * p.n_mt;
            uphase = (uint32_t)u & 1u;
            int dummy;
            if (!walk.seek<TILE_N>(blockIdx.x + (long long)u * gridDim.x, dummy, nt)) break;
          } else if (!walk.seek<TILE_N>(blockIdx.x + (long long)n * gridDim.x, mt, nt)) {
            break;
          }
          cur_n = n;
          e = walk.e;
          n0 = nt * TILE_N;
          if (!tile_role) {
            sfb_base = p.sfb + (((long long)e * p.sfb_rt + (n0 >> 7)) * p.n_kt) * 512;
            sfb_row_atoms = TILE_N > 128 ? min(2, p.sfb_rt - (n0 >> 7)) : 1;
            e_base = p.e_meta + (((long long)e * p.e_k_atoms) * p.e_m_atoms + mt) * 2048;
            sfa_base = p.sfa + (((long long)e * p.n_mt + mt) * p.n_kt) * 512;
          }
        }
        const int k_atoms = min(C::kAtoms, p.n_kt - ks * C::kAtoms);
        const int b_boxes = (k_atoms + 1) / 2;
        if (kBRes && tile_role && mt == 0) {
          // this unit's activation chunks of this stage, as soon as the previous unit has finished with them
          if (!ptx::mbar_wait(b_empty + ks, uphase ^ 1)) {
            atomicExch(&g_status, kProducerEmptyTimeout);
            ok = false;
            break;
          }
          uint8_t* dst = b_res + ks * (C::kBBoxes * C::kBBoxBytes);
          if (p.b_4d) {
            ptx::mbar_arrive_expect_tx(b_full + ks, C::kBBoxes * C::kBBoxBytes);
            ptx::tma_load_4d(dst, &map_b, b_full + ks, 0, n0, ks * C::kBBoxes, e);
          } else {
            ptx::mbar_arrive_expect_tx(b_full + ks, b_boxes * C::kBBoxBytes);
            for (int b = 0; b < b_boxes; ++b)
              ptx::tma_load_3d(dst + b * C::kBBoxBytes, &map_b, b_full + ks, (ks * C::kBBoxes + b) * 128, n0, e);
          }
        }
        long long tq0 = p.prof ? clock64() : 0;
        if (!ptx::mbar_wait(empty_bar + stage, turn ^ 1u)) {
          atomicExch(&g_status, tile_role ? kProducerEmptyTimeout : kSideProducerTimeout);
          ok = false;
          break;
        }
        if (p.prof && threadIdx.x == 0) p.prof[blockIdx.x * 8 + 4] += clock64() - tq0;
        uint8_t* st = stage_base + stage * C::kStageBytes;
        if (tile_role) {
          // with the 4-D activation map one copy fetches all of the stage's 256-K chunks (a box past the
          // last chunk is zero-filled and still counts its full size)
          const int b_bytes = kBRes ? 0 : (p.b_4d ? C::kBBoxes : b_boxes) * C::kBBoxBytes;
          ptx::mbar_arrive_expect_tx(full_bar + stage, C::kABytes + b_bytes);
          ptx::tma_load_3d(st + C::kOffA, &map_a, full_bar + stage, ks * C::kARowBytes, mt * kTileM, e);
          if (!kBRes) {
            if (p.b_4d) {
              ptx::tma_load_4d(st + C::kOffB, &map_b, full_bar + stage, 0, n0, ks * C::kBBoxes, e);
            } else {
              for (int b = 0; b < b_boxes; ++b)
                ptx::tma_load_3d(st + C::kOffB + b * C::kBBoxBytes, &map_b, full_bar + stage,
                                 ks * (STAGE_K / 2) + b * 128, n0, e);
            }
          }
        } else {
          const int e_atoms = (k_atoms + 1) / 2;
          const uint32_t sf_bytes = 512u * k_atoms;
          if (part == 0) {
            ptx::mbar_arrive_expect_tx(full_bar + stage, e_atoms * 2048);
            for (int ea = 0; ea < e_atoms; ++ea)
              ptx::bulk_load(st + C::kOffE + ea * 2048,
                             e_base + (long long)(ks * C::kEAtoms + ea) * p.e_m_atoms * 2048, 2048, full_bar + stage);
          } else {
            ptx::mbar_arrive_expect_tx(full_bar + stage, sf_bytes * (1 + sfb_row_atoms));
            ptx::bulk_load(st + C::kOffSfa, sfa_base + ks * (C::kAtoms * 512), sf_bytes, full_bar + stage);
            for (int ra = 0; ra < sfb_row_atoms; ++ra)
              ptx::bulk_load(st + C::kOffSfb + ra * C::kSfaBytes,
                             sfb_base + ((long long)ra * p.n_kt + ks * C::kAtoms) * 512, sf_bytes, full_bar + stage);
          }
        }
        ks += p.prod_lanes;
        stage += p.prod_lanes;
        if (stage >= p.stages) { stage -= p.stages; turn ^= 1u; }
      }
      if (!ok) {
        // give copies already in flight time to land before the CTA's shared memory is released
#pragma unroll 1
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 2 || warp == 3) {
    // =============================== MMA issuers ===============================
    // A tcgen05.mma holds its issuing thread for about as long as it executes, so whatever else
    // that thread does between two MMAs (waits, descriptor arithmetic, commits: a few hundred
    // cycles per stage for a lone thread) is time the tensor pipe idles.  Two issuers in two warps
    // take alternate tiles, each into its own accumulator stage; while one is between MMAs the
    // other's are executing.  Every tile's MMAs still come from one thread, in K order.
    constexpr int kIssuers = (C::kAccStages == 2 && !kBRes) ? 2 : 1;
    const int issuer = warp - 2;
    const int n_items = my_work_items<TILE_N>(s_counts, p.E, kBRes ? 1 : p.n_mt, lane);
    if (lane == 0 && issuer < kIssuers) {
      constexpr uint32_t idesc = ptx::mma_sp_nvf4_idesc(TILE_N);
      int stage = 0, acc = kIssuers == 2 ? issuer : 0;
      uint32_t phase = 0, acc_phase = 0, uphase = 0, soff = 0;
      bool ok = true;
      long long c_wait_sf = 0, c_issue = 0, c_wait_acc = 0, n_stage = 0;
      const bool prof = p.prof != nullptr && issuer == 0;
      // Pass over the stages of a tile the other issuer takes.  Each one is waited for, not just
      // counted: a parity wait only tells two consecutive phases of a barrier apart, so an issuer
      // must see every turn of every slot, or after a long tile it would take an old phase for its own.
      auto skip_stages = [&](int n) {
#pragma unroll 1
        for (int i = 0; i < n && ok; ++i) {
          if (!ptx::mbar_wait(sf_full + stage, phase)) {
            atomicExch(&g_status, kMmaScaleTimeout);
            ok = false;
          }
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        soff = (uint32_t)stage * (C::kStageBytes >> 4);
      };
      if (kIssuers == 2 && issuer == 1 && n_items > 1) skip_stages(p.k_stages);
      const long long t_begin = prof ? clock64() : 0;
      unsigned long long ns_begin = 0;
      if (prof) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns_begin));
      // stage-0 descriptors, split into the 32-bit halves: only the low half changes with the address
      const uint64_t d_a0 = ptx::smem_desc(ptx::smem_u32(stage_base) + C::kOffA, 8 * C::kARowBytes, 16, C::kASwizzle);
      const uint64_t d_b0 = ptx::smem_desc(kBRes ? ptx::smem_u32(b_res) : ptx::smem_u32(stage_base) + C::kOffB, 1024, 16, 2);
      const uint64_t d_e0 = ptx::smem_desc(ptx::smem_u32(stage_base) + C::kOffE, 128, 0, 0);
      const uint32_t lo_a0 = (uint32_t)d_a0, hi_a = (uint32_t)(d_a0 >> 32);
      const uint32_t lo_b0 = (uint32_t)d_b0, hi_b = (uint32_t)(d_b0 >> 32);
      const uint32_t lo_e0 = (uint32_t)d_e0, hi_e = (uint32_t)(d_e0 >> 32);
      const uint32_t e_cols = tmem_base + C::kColE + issuer * (4 * C::kEAtoms);   // private metadata columns
      const uint32_t sf_cols0 = tmem_base + C::kColSf;
      const int tiles_per_item = kBRes ? p.n_mt : 1;
      const int last_atoms = p.n_kt - (p.k_stages - 1) * C::kAtoms;     // K-blocks of a tile's last stage
      for (int item = kIssuers == 2 ? issuer : 0; item < n_items && ok; item += kIssuers) {
        // a 64-wide tile's scales sit 0 or 2 columns into the 128-row atom (even offsets only: the MMA
        // faults on an odd scale column); wider tiles start at column 0 and need no tile coordinates
        uint32_t sfb_off = 0;
        if (TILE_N < 128) {
          int mt_lo, mt_hi, nt;
          if (!next_work<TILE_N, kBRes>(walk, blockIdx.x + (long long)item * gridDim.x, p.n_mt, mt_lo, mt_hi, nt)) break;
          sfb_off = ((nt * TILE_N) & 127) >> 5;
        }
        for (int mt = 0; mt < tiles_per_item && ok; ++mt) {
          long long tp0 = prof ? clock64() : 0;
          if (!ptx::mbar_wait(acc_empty + acc, acc_phase ^ 1)) {
            atomicExch(&g_status, kMmaAccTimeout);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          if (prof) c_wait_acc += clock64() - tp0;
          const uint32_t d_tmem = tmem_base + acc * TILE_N;
#pragma unroll 1
          for (int ks = 0; ks < p.k_stages; ++ks) {
            long long tp1 = prof ? clock64() : 0;
            const int k_atoms = ks + 1 == p.k_stages ? last_atoms : C::kAtoms;
            if (kBRes && mt == 0 && !ptx::mbar_wait(b_full + ks, uphase)) {
              atomicExch(&g_status, kMmaFullTimeout);
              ok = false;
              break;
            }
            if (!ptx::mbar_wait(sf_full + stage, phase)) {
              atomicExch(&g_status, kMmaScaleTimeout);
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            long long tp3 = prof ? clock64() : 0;
            if (prof) { c_wait_sf += tp3 - tp1; ++n_stage; }
            // descriptors of this stage: the precomputed ones of stage 0 plus the stage's offset in
            // 16-byte units (the address field is the low 14 bits, so a 32-bit add cannot carry out)
            const uint32_t la = lo_a0 + soff, le = lo_e0 + soff;
            const uint32_t lb = kBRes ? lo_b0 + ks * ((C::kBBoxes * C::kBBoxBytes) >> 4) : lo_b0 + soff;
            const uint32_t sf_cols = sf_cols0 + stage * C::kSfSlotCols;
            const uint32_t sfb_cols = sf_cols + C::kAtoms * 4 + sfb_off;
            if (k_atoms == C::kAtoms) {
#pragma unroll
              for (int ea = 0; ea < C::kEAtoms; ++ea) ptx::tc_cp_128x128b(e_cols + ea * 4, pack_desc(le + ea * 128, hi_e));
#pragma unroll
              for (int ka = 0; ka < C::kAtoms; ++ka)
                ptx::tc_mma_sp_nvf4(d_tmem, pack_desc(la + ka * 2, hi_a),
                                    pack_desc(lb + (ka >> 1) * (C::kBBoxBytes >> 4) + (ka & 1) * 4, hi_b), idesc,
                                    (ks | ka) != 0 ? 1u : 0u, sf_cols + ka * 4, sfb_cols + ka * C::kSfbColsPerAtom,
                                    e_cols + ka * 2);
            } else {
#pragma unroll
              for (int ea = 0; ea < C::kEAtoms; ++ea)
                if (2 * ea < k_atoms) ptx::tc_cp_128x128b(e_cols + ea * 4, pack_desc(le + ea * 128, hi_e));
#pragma unroll
              for (int ka = 0; ka < C::kAtoms; ++ka)
                if (ka < k_atoms)
                  ptx::tc_mma_sp_nvf4(d_tmem, pack_desc(la + ka * 2, hi_a),
                                      pack_desc(lb + (ka >> 1) * (C::kBBoxBytes >> 4) + (ka & 1) * 4, hi_b), idesc,
                                      (ks | ka) != 0 ? 1u : 0u, sf_cols + ka * 4, sfb_cols + ka * C::kSfbColsPerAtom,
                                      e_cols + ka * 2);
            }
            ptx::tc_commit(empty_bar + stage);   // stage and scale slot reusable once these MMAs and copies retire
            if (kBRes && mt + 1 == tiles_per_item) ptx::tc_commit(b_empty + ks);   // last weight tile: chunks may be replaced
            if (prof) c_issue += clock64() - tp3;
            soff += C::kStageBytes >> 4;
            if (++stage == p.stages) { stage = 0; soff = 0; phase ^= 1; }
          }
          if (!ok) break;
          ptx::tc_commit(acc_full + acc);
          if (kIssuers == 2) {
            acc_phase ^= 1;                 // this issuer's accumulator stage comes round every own tile
            if (item + kIssuers < n_items) skip_stages(p.k_stages);
          } else if (++acc == C::kAccStages) {
            acc = 0;
            acc_phase ^= 1;
          }
        }
        uphase ^= 1;
      }
      if (prof) {
        long long* q = p.prof + blockIdx.x * 8;
        q[0] = 0; q[1] = c_issue; q[2] = c_wait_acc; q[3] = n_stage; q[5] = c_wait_sf;
        unsigned long long ns_end;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns_end));
        long long* x = p.prof + 256 * 8 + blockIdx.x * 8;   // issuer loop: cycles and nanoseconds
        if (!kFused) { x[0] = clock64() - t_begin; x[1] = (long long)(ns_end - ns_begin); }
      }
    }
    __syncwarp();
  } else if (warp < 8) {
    // =============================== scale loaders ===============================
    const int n_items = my_work_items<TILE_N>(s_counts, p.E, kBRes ? 1 : p.n_mt, lane);
    const long long n_stages = (long long)n_items * (kBRes ? p.n_mt : 1) * p.k_stages;
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + C::kColSf;
    int stage = 0;
    uint32_t phase = 0;
#pragma unroll 1
    const bool lprof = p.prof != nullptr && warp == 4 && lane == 0;
    long long l_wait = 0, l_work = 0;
    for (long long g = 0; g < n_stages; ++g) {
      long long tl0 = lprof ? clock64() : 0;
      if (!ptx::mbar_wait(full_bar + stage, phase)) {
        atomicExch(&g_status, kScaleLoaderTimeout);
        break;
      }
      long long tl1 = lprof ? clock64() : 0;
      const uint8_t* st = stage_base + stage * C::kStageBytes + lane * 16;
      const uint32_t cols = lane_base + stage * C::kSfSlotCols;
#pragma unroll
      for (int ka = 0; ka < C::kAtoms; ++ka) {
        ptx::tc_st_32x32_x4(cols + ka * 4, *reinterpret_cast<const uint4*>(st + C::kOffSfa + ka * 512));
#pragma unroll
        for (int ra = 0; ra < C::kSfbRowAtoms; ++ra)
          ptx::tc_st_32x32_x4(cols + C::kAtoms * 4 + ka * C::kSfbColsPerAtom + ra * 4,
                              *reinterpret_cast<const uint4*>(st + C::kOffSfb + ra * C::kSfaBytes + ka * 512));
      }
      ptx::tc_st_wait();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        ptx::mbar_arrive(sf_full + stage);
        ptx::mbar_arrive(empty_bar + stage);   // the scales have left shared memory
      }
      if (lprof) { l_wait += tl1 - tl0; l_work += clock64() - tl1; }
      if (++stage == p.stages) { stage = 0; phase ^= 1; }
    }
    if (lprof) {   // scale loader: waiting for a stage to land, moving its scales
      p.prof[256 * 8 + blockIdx.x * 8 + 6] = l_wait;
      p.prof[256 * 8 + blockIdx.x * 8 + 7] = l_work;
    }
  } else {
    // =============================== epilogue ===============================
    const int group = (warp - 8) >> 2;         // chunks of 32 token columns alternate between the groups
    const int sub = warp & 3;                  // tensor-memory lane quarter this warp may read
    const int ep_tid = threadIdx.x - 256 - group * 128;
    const int m_local = sub * 32 + lane;       // accumulator row (output feature) held by this thread
    const bool vec_ok = (p.M % 8) == 0;        // 16-byte stores need 16-byte aligned output rows
    __nv_bfloat16* group_out = s_out + group * (2 * 32 * kOutRow);
    int acc = 0;
    uint32_t acc_phase = 0, chunk = 0;
    if (kFused) {
      // Benign fill of GEMM2's scale buffer: every byte the epilogues will not write (rows at or
      // past counts[e], K-block slop) becomes 0x38.  All CTAs share the lines; live slots are
      // skipped, so the fill never races with a quantized scale.
      const int KB = p.f_n / kSfBlock;
      const unsigned lines = (unsigned)p.E * p.sfb_rt * p.f_n_kt * 32u;   // < 2^27, checked by the host
      const uint32_t w4 = kBenignSf * 0x01010101u;
#pragma unroll 1
      for (unsigned c = blockIdx.x * 256 + (threadIdx.x - 256); c < lines; c += gridDim.x * 256) {
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
    bool ok = true;
    for (long long w = blockIdx.x; ok; w += gridDim.x) {
      int mt_lo, mt_hi, nt;
      if (!next_work<TILE_N, kBRes>(walk, w, p.n_mt, mt_lo, mt_hi, nt)) break;
      const int e = walk.e;
      const int cnt = s_counts[e];
      const float alpha = p.alphas[e];
      float gs = 0.f;
      if (kFused) gs = p.f_gpe ? p.f_gscale[e] : p.f_gscale[0];
      const int n0 = nt * TILE_N;
      __nv_bfloat16* out_e = p.out + (long long)e * p.max_n * p.M;
      for (int mt = mt_lo; mt < mt_hi; ++mt) {
      const bool eprof = p.prof != nullptr && ep_tid == 0 && group == 0;
      long long te0 = eprof ? clock64() : 0;
      if (!ptx::mbar_wait(acc_full + acc, acc_phase)) {
        atomicExch(&g_status, kEpilogueTimeout);
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      long long te1 = eprof ? clock64() : 0;
      if (!kFused) {
        // Plain epilogue, warp by warp with no barrier between warps: 32 token columns at a time are
        // scaled, rounded, transposed through the warp's own corner of shared memory ([32 tokens][32
        // features], rows padded to 80 bytes) and stored 16 bytes per lane, 64 contiguous bytes per
        // output row.  (Waiting for the tensor-memory load is a negligible part of the time, so the
        // loads are not double buffered; registers go to the wider piece instead.)
        constexpr int kWarpRow = 40;
        __nv_bfloat16* buf = s_out + (warp - 8) * (32 * kWarpRow);
        const uint32_t t_row = tmem_base + ((uint32_t)(sub * 32) << 16) + acc * TILE_N;
        const int m = mt * kTileM + sub * 32 + (lane & 3) * 8;
        long long t_w = 0;
#pragma unroll 1
        for (int c = group * 32; c < TILE_N && n0 + c < cnt; c += 64) {
          uint32_t v[32];
          long long tq = eprof ? clock64() : 0;
          ptx::tc_ld_32x32(t_row + c, v);
          ptx::tc_ld_wait();
          if (eprof) t_w += clock64() - tq;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            buf[i * kWarpRow + lane] = __float2bfloat16_rn(__fmul_rn(alpha, __uint_as_float(v[i])));
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int tok = (lane >> 2) + 8 * j;
            const int n = n0 + c + tok;
            if (n >= cnt || m >= p.M) continue;
            const __nv_bfloat16* src = buf + tok * kWarpRow + (lane & 3) * 8;
            if (vec_ok) {
              *reinterpret_cast<uint4*>(out_e + (long long)n * p.M + m) = *reinterpret_cast<const uint4*>(src);
            } else {
#pragma unroll 1
              for (int z = 0; z < 8 && m + z < p.M; ++z) out_e[(long long)n * p.M + m + z] = src[z];
            }
          }
          __syncwarp();   // the next piece overwrites the buffer
        }
        if (eprof) p.prof[256 * 8 + blockIdx.x * 8 + 5] += t_w;   // waiting for tensor-memory loads
      }
#pragma unroll 1
      for (int c0 = group * 32; kFused && c0 < TILE_N; c0 += 64) {
        if (n0 + c0 >= cnt) break;             // uniform over the group's four warps
        uint32_t r[32];
        ptx::tc_ld_32x32(tmem_base + ((uint32_t)(sub * 32) << 16) + acc * TILE_N + c0, r);
        ptx::tc_ld_wait();
        __nv_bfloat16* buf = group_out + (chunk & 1) * (32 * kOutRow);
        ++chunk;
        {
          // The weight rows are interleaved in 64-row blocks (32 gate rows, then the 32 matching up
          // rows), so lanes of the even 32-lane quarters hold gates and the odd quarters the ups of
          // the same 32 output features: exactly one quantization block per token.  Every lane parks
          // its values; the gate lane of a feature then finishes the even token columns and the up
          // lane the odd ones, leaving the product in the gate's slot.
          long long tf0 = eprof ? clock64() : 0;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            buf[i * kOutRow + m_local] = __float2bfloat16_rn(__fmul_rn(alpha, __uint_as_float(r[i])));
          long long tf1 = eprof ? clock64() : 0;
          epilogue_pair_sync(group, sub);
          long long tf2 = eprof ? clock64() : 0;
          const bool is_up = (sub & 1) != 0;
          __nv_bfloat16* col0 = buf + (is_up ? kOutRow + m_local - 32 : m_local);
          if (p.f_act.kind == PNV_ACT_SILU && p.f_act.silu_tab != nullptr) {
            // SiLU through the table: all 16 columns of this lane in one straight-line pass (16 independent
            // loads of the table in flight)
            float g[16], u[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              g[i] = __bfloat162float(col0[i * 2 * kOutRow]);
              u[i] = __bfloat162float(col0[i * 2 * kOutRow + 32]);
            }
            float sv[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) sv[i] = silu_lookup(g[i], p.f_act.silu_tab);
#pragma unroll
            for (int i = 0; i < 16; ++i) col0[i * 2 * kOutRow] = __float2bfloat16_rn(__fmul_rn(sv[i], u[i]));
          } else {
#pragma unroll 1
            for (int i0 = 0; i0 < 16; i0 += 8) {
              float g[8], u[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                g[i] = __bfloat162float(col0[(i0 + i) * 2 * kOutRow]);
                u[i] = __bfloat162float(col0[(i0 + i) * 2 * kOutRow + 32]);
              }
              __nv_bfloat16 y[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) y[i] = __float2bfloat16_rn(gated_act(g[i], u[i], p.f_act));
#pragma unroll
              for (int i = 0; i < 8; ++i) col0[(i0 + i) * 2 * kOutRow] = y[i];
            }
          }
          long long tf3 = eprof ? clock64() : 0;
          epilogue_pair_sync(group, sub);
          long long tf4 = eprof ? clock64() : 0;
          // quantize: two adjacent lanes share one (token, 32-feature block); each takes 16 features
          const int pair = ep_tid >> 1, hb = ep_tid & 1;
          const int i = pair & 31, blk = pair >> 5;
          const int n = n0 + c0 + i;
          const uint4* src = reinterpret_cast<const uint4*>(buf + i * kOutRow + blk * 64 + hb * 16);
          float f[2][8];
          float amax = 0.f;
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            unpack8(src[q], f[q]);
#pragma unroll
            for (int z = 0; z < 8; ++z) amax = fmaxf(amax, fabsf(f[q][z]));
          }
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
          uint32_t sf_byte;
          float inv;
          block_scale(amax, gs, sf_byte, inv);
          if (n < cnt) {
            const int kb = mt * 2 + blk;       // 32-feature block of the N-wide output
            const long long row = (long long)e * p.max_n + n;
            *reinterpret_cast<uint2*>(p.f_b_out + row * (p.f_n / 2) + kb * 16 + hb * 8) =
                make_uint2(quant8(f[0], inv), quant8(f[1], inv));
            if (hb == 0) p.f_sfb_out[sf_offset(e, n, kb, p.sfb_rt, p.f_n_kt)] = (uint8_t)sf_byte;
          }
          if (eprof) {   // fused epilogue phases: park, first barrier, gate math, second barrier, quantize
            long long* x = p.prof + 256 * 8 + blockIdx.x * 8;
            x[0] += tf1 - tf0; x[1] += tf2 - tf1; x[2] += tf3 - tf2; x[3] += tf4 - tf3; x[4] += clock64() - tf4;
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(acc_empty + acc);
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
      if (eprof) {   // waiting for an accumulator, and group 0's share of the tile's epilogue
        long long* q = p.prof + blockIdx.x * 8;
        q[6] += te1 - te0; q[7] += clock64() - te1;
      }
      }
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

// 3-D byte tensor [experts][rows][row_bytes] with a [1][box_rows][box_bytes] box.
// 4-D view of the activations [experts][K/256 chunks][rows][128 B] for K a multiple of 256: one box
// [chunks][box_rows][128 B] is `chunks` consecutive 128-byte-swizzled operand tiles in shared memory.
int make_map_b4(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t experts,
                uint32_t box_rows, uint32_t box_chunks) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(PNV_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[4] = {128, rows, row_bytes / 128, experts};
  cuuint64_t strides[3] = {row_bytes, 128, row_bytes * rows};
  cuuint32_t box[4] = {128, box_rows, box_chunks, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(PNV_ERR_CUDA, "cuTensorMapEncodeTiled (4-D) failed with CUresult %d (row_bytes=%llu rows=%llu)",
                (int)r, (unsigned long long)row_bytes, (unsigned long long)rows);
  return PNV_OK;
}

int make_map(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t experts,
             uint32_t box_bytes, uint32_t box_rows, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(PNV_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {row_bytes, rows, experts};
  cuuint64_t strides[2] = {row_bytes, row_bytes * rows};
  cuuint32_t box[3] = {box_bytes, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(PNV_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (row_bytes=%llu rows=%llu)",
                (int)r, (unsigned long long)row_bytes, (unsigned long long)rows);
  return PNV_OK;
}

// Traced build: breadcrumb buffer in host-mapped memory, enabled with PNV_GROUP_MM_TRACE=1.
constexpr int kTraceWords = 8 * 16;
unsigned* g_trace_host = nullptr;   // host view
unsigned* g_trace_dev = nullptr;    // device view of the same pages

// PNV_GROUP_MM_PROFILE=1: the MMA issuer and the tile producer of every CTA accumulate cycle
// counters (waiting for data, issuing, waiting for an accumulator, stages; waiting for a free
// stage) in a device buffer that pnv_group_mm_profile() reads back.  A measuring aid only.
long long* g_prof_dev = nullptr;
long long* profile_buffer(bool fused) {   // PNV_GROUP_MM_PROFILE=2 records the fused launches only
  static int v = -1;
  if (v < 0) {
    const char* env = std::getenv("PNV_GROUP_MM_PROFILE");
    v = (env != nullptr && (env[0] == '1' || env[0] == '2')) ? env[0] - '0' : 0;
  }
  if (v == 0 || (v == 2 && !fused)) return nullptr;
  if (g_prof_dev == nullptr) {
    if (cudaMalloc(reinterpret_cast<void**>(&g_prof_dev), 256 * 16 * sizeof(long long)) != cudaSuccess) return nullptr;
  }
  cudaMemset(g_prof_dev, 0, 256 * 16 * sizeof(long long));
  return g_prof_dev;
}

bool trace_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* env = std::getenv("PNV_GROUP_MM_TRACE");
    v = (env != nullptr && env[0] == '1') ? 1 : 0;
  }
  return v == 1;
}

template <int TILE_N, int STAGE_K, int ISSUERS, bool kTrace, bool kFused>
int launch_impl(const CUtensorMap& map_a, const CUtensorMap& map_b, const Params& p_in, int sm_count, bool pdl,
                cudaStream_t stream) {
  using C = Cfg<TILE_N, STAGE_K, ISSUERS>;
  Params p = p_in;
  p.stages = C::kStages;
  if (const char* env = std::getenv("PNV_GROUP_MM_STAGES")) {   // experiment knob: shallower pipeline
    int v = std::atoi(env);
    if (v >= 1 && v < C::kStages) p.stages = v;
  }
  const size_t smem = 1024 + (size_t)C::kStages * C::kStageBytes + kOutStageBytes + 256 + 4 * (size_t)p.E;
  static_assert(kOutStageBytes % 16 == 0, "barrier block must stay aligned");
  static_assert(8 * (2 * C::kStages + 2 * C::kAccStages + 2 + ISSUERS) + 16 <= 256, "barrier block overflows its slot");
  // opt in to the large dynamic shared-memory carve-out once per device
  static bool opted_in[64] = {};
  int dev = 0;
  PNV_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !opted_in[dev]) {
    PNV_CUDA(cudaFuncSetAttribute(group_mm_kernel<TILE_N, STAGE_K, ISSUERS, kTrace, kFused>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    if (dev >= 0 && dev < 64) opted_in[dev] = true;
  }
  long long max_tiles = (long long)p.E * p.n_mt * ceil_div_i(p.max_n, TILE_N);
  int grid = (int)(max_tiles < sm_count ? max_tiles : sm_count);
  if (grid < 1) grid = 1;
  PNV_CUDA(launch_pdl(group_mm_kernel<TILE_N, STAGE_K, ISSUERS, kTrace, kFused>, dim3(grid), dim3(C::kThreads), smem,
                      stream, pdl, map_a, map_b, p));
  return PNV_OK;
}

template <int TILE_N, int STAGE_K, int ISSUERS>
int launch(const CUtensorMap& map_a, const CUtensorMap& map_b, Params& p, int sm_count, bool pdl,
           cudaStream_t stream) {
  if (p.f_b_out != nullptr) {
    p.trace = nullptr;
    return launch_impl<TILE_N, STAGE_K, ISSUERS, false, true>(map_a, map_b, p, sm_count, pdl, stream);
  }
  if (!trace_enabled()) {
    p.trace = nullptr;
    return launch_impl<TILE_N, STAGE_K, ISSUERS, false, false>(map_a, map_b, p, sm_count, pdl, stream);
  }
  if (g_trace_host == nullptr) {
    PNV_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&g_trace_host), kTraceWords * sizeof(unsigned),
                           cudaHostAllocMapped));
    PNV_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&g_trace_dev), g_trace_host, 0));
  }
  for (int i = 0; i < kTraceWords; ++i) g_trace_host[i] = 0;
  p.trace = g_trace_dev;
  return launch_impl<TILE_N, STAGE_K, ISSUERS, true, false>(map_a, map_b, p, sm_count, false, stream);
}

// PNV_GROUP_MM_BRES=1 keeps the activation tile resident whenever it fits; otherwise it is streamed.
int bres_mode() {
  static int v = -2;
  if (v == -2) {
    const char* env = std::getenv("PNV_GROUP_MM_BRES");
    v = env == nullptr ? -1 : (env[0] == '0' ? 0 : 1);
  }
  return v;
}

template <int TILE_N, int STAGE_K, bool kFused, bool kBRes>
int launch_wide_impl(const CUtensorMap& map_a, const CUtensorMap& map_b, const Params& p_in, int sm_count, bool pdl,
                     cudaStream_t stream, int stages, int b_res_bytes) {
  using C = WideCfg<TILE_N, STAGE_K, kBRes>;
  Params p = p_in;
  p.stages = stages;
  if (const char* env = std::getenv("PNV_GROUP_MM_STAGES")) {   // experiment knob: shallower pipeline
    const int v = std::atoi(env);
    if (v >= 2 && v < stages) p.stages = stages = v;
  }
  p.b_res_bytes = b_res_bytes;
  p.prod_lanes = stages >= 8 ? 4 : stages >= 4 ? 2 : 1;
  if (const char* env = std::getenv("PNV_GROUP_MM_LANES")) {   // experiment knob
    const int v = std::atoi(env);
    if (v >= 1 && v <= 16) p.prod_lanes = std::min(v, stages);
  }
  // resident mode: a lane must never wait for a chunk that a later lane of the same batch releases
  if (kBRes) p.prod_lanes = std::max(1, std::min(p.prod_lanes, p.k_stages));
  p.trace = nullptr;
  const size_t smem = 1024 + (size_t)b_res_bytes + (size_t)stages * C::kStageBytes +
                      (kFused ? C::kOutBytes : C::kPlainOutBytes) + C::kBarrierBytes + 4 * (size_t)p.E;
  static bool opted_in[64] = {};
  int dev = 0;
  PNV_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !opted_in[dev]) {
    PNV_CUDA(cudaFuncSetAttribute(group_mm_wide_kernel<TILE_N, STAGE_K, kFused, kBRes>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    if (dev >= 0 && dev < 64) opted_in[dev] = true;
  }
  const long long units = (long long)p.E * ceil_div_i(p.max_n, TILE_N);
  const long long max_work = kBRes ? units : units * p.n_mt;
  int grid = (int)(max_work < sm_count ? max_work : sm_count);
  if (grid < 1) grid = 1;
  PNV_CUDA(launch_pdl(group_mm_wide_kernel<TILE_N, STAGE_K, kFused, kBRes>, dim3(grid), dim3(C::kThreads), smem,
                      stream, pdl, map_a, map_b, p));
  return PNV_OK;
}

template <int TILE_N, int STAGE_K>
int launch_wide(const CUtensorMap& map_a, const CUtensorMap& map_b, Params& p, int sm_count, bool pdl,
                cudaStream_t stream) {
  using CS = WideCfg<TILE_N, STAGE_K, false>;
  using CR = WideCfg<TILE_N, STAGE_K, true>;
  const bool fused = p.f_b_out != nullptr;
  const int fixed = 1024 + (fused ? CS::kOutBytes : CS::kPlainOutBytes) + CS::kBarrierBytes + 4 * p.E;
  // resident activation tile: one slab of TILE_N x STAGE_K / 2 bytes per K stage, and still two stages of weights
  const int b_res = p.k_stages * CR::kBBoxes * CR::kBBoxBytes;
  const int stages_res = std::min(std::min((int)CR::kMaxStages, (int)CR::kSfSlots), (kSmemLimit - fixed - b_res) / CR::kStageBytes);
  const long long units = (long long)p.E * ceil_div_i(p.max_n, TILE_N);
  const bool fits = p.k_stages <= CR::kMaxChunks && b_res < kSmemLimit - fixed && stages_res >= 2;
  (void)units;   // resident mode is opt-in (PNV_GROUP_MM_BRES=1) until it measures faster than streaming
  const bool resident = fits && bres_mode() == 1;
  if (resident) {
    if (fused) return launch_wide_impl<TILE_N, STAGE_K, true, true>(map_a, map_b, p, sm_count, pdl, stream, stages_res, b_res);
    return launch_wide_impl<TILE_N, STAGE_K, false, true>(map_a, map_b, p, sm_count, pdl, stream, stages_res, b_res);
  }
  const int stages = std::min(std::min((int)CS::kMaxStages, (int)CS::kSfSlots), (kSmemLimit - fixed) / CS::kStageBytes);
  if (stages < 2) return fail(PNV_ERR_INVALID_ARGUMENT, "group_mm: not enough shared memory for a %dx%d pipeline", TILE_N, STAGE_K);
  if (fused) return launch_wide_impl<TILE_N, STAGE_K, true, false>(map_a, map_b, p, sm_count, pdl, stream, stages, 0);
  return launch_wide_impl<TILE_N, STAGE_K, false, false>(map_a, map_b, p, sm_count, pdl, stream, stages, 0);
}

// Tile variants.  The first eight names and ids are the reference's; a "2sm" name is accepted with
// its cluster rule and runs the same one-CTA tiles as its "1sm" sibling; "_k512" selects 512-K
// pipeline stages (128-byte weight rows per TMA box) instead of 256-K stages.
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

extern "C" int pnv_group_mm_profile(long long* out, int n_values) {
  PNV_REQUIRE(out && n_values >= 0 && n_values <= 256 * 16, "bad profile buffer");
  PNV_REQUIRE(g_prof_dev != nullptr, "profiling is off: set PNV_GROUP_MM_PROFILE=1 before the first group_mm");
  PNV_CUDA(cudaDeviceSynchronize());
  PNV_CUDA(cudaMemcpy(out, g_prof_dev, n_values * sizeof(long long), cudaMemcpyDeviceToHost));
  return PNV_OK;
}

extern "C" int pnv_group_mm_debug_trace(unsigned* words_out, int n_words) {
  PNV_REQUIRE(words_out && n_words >= 0, "bad trace buffer");
  for (int i = 0; i < n_words; ++i)
    words_out[i] = (g_trace_host != nullptr && i < kTraceWords) ? ((volatile unsigned*)g_trace_host)[i] : 0u;
  return PNV_OK;
}

namespace pnv {
namespace {

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
};
constexpr int kNumFusedKinds = sizeof(kFusedKinds) / sizeof(kFusedKinds[0]);

int group_mm_common(void* out, const FusedArgs* fused, const uint8_t* a_comp, const uint8_t* e_meta,
                    const uint8_t* sfa, const uint8_t* b_act, const uint8_t* sfb, const float* alphas,
                    const int32_t* counts, int experts, int features, int k, int max_n, int config_id,
                    int cluster_m, int cluster_n, int sm_count, int pdl, pnv_stream_t stream,
                    const char* display_name) {
  PNV_REQUIRE(out && a_comp && e_meta && sfa && b_act && sfb && alphas && counts, "null pointer argument");
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
  p.f_b_out = nullptr; p.f_sfb_out = nullptr; p.f_gscale = nullptr; p.f_gpe = 0; p.f_n = 0; p.f_n_kt = 0;
  p.f_act = GatedAct{PNV_ACT_SILU, 1.f, -1.f, nullptr};
  if (fused != nullptr) {
    p.f_b_out = fused->b_out; p.f_sfb_out = fused->sfb_out; p.f_gscale = fused->gscale; p.f_gpe = fused->gpe;
    p.f_n = features / 2; p.f_n_kt = sf_k_atoms(features / 2); p.f_act = fused->act;
  }
  p.E = experts; p.M = features; p.K = k; p.max_n = max_n;
  p.n_mt = ceil_div_i(features, kTileM);
  p.k_stages = ceil_div_i(k, kind.stage_k);
  p.n_kt = sf_k_atoms(k);
  p.e_k_atoms = wd.k_e / 16;
  p.e_m_atoms = wd.m_e / 128;
  p.sfb_rt = sf_row_atoms(max_n);
  const char* only_m = std::getenv("PNV_GROUP_MM_PROFILE_M");   // record only launches with this many features
  p.prof = (only_m != nullptr && std::atoi(only_m) != features) ? nullptr : profile_buffer(fused != nullptr);
  p.stages = 0;
  p.b_res_bytes = 0;
  p.b_4d = 0;
  p.prod_lanes = 1;
  p.trace = nullptr;

  // Tile geometry.  The variant names fix the widest token tile; when every expert's tokens fit one
  // narrow tile (max_n <= 32) the kernel runs 16- or 32-wide MMAs over 512-K stages with four issuer
  // warps instead: same results, far less padding and a deeper pipeline.
  int tile_n = kind.tile_n, stage_k = kind.stage_k;
  static const bool narrow_ok = [] {
    const char* env = std::getenv("PNV_GROUP_MM_NARROW");
    return !(env != nullptr && env[0] == '0');
  }();
  if (narrow_ok && max_n <= 32) {
    tile_n = max_n <= 16 ? 16 : 32;
    stage_k = 512;
  }
  p.k_stages = ceil_div_i(k, stage_k);

  CUtensorMap map_a, map_b;
  if (int rc = make_map(&map_a, a_comp, (uint64_t)wd.k_ac / 2, (uint64_t)wd.m_ac, (uint64_t)experts,
                        (uint32_t)stage_k / 4, (uint32_t)kTileM,
                        stage_k == 512 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B))
    return rc;
  static const bool wide_ok = [] {   // PNV_GROUP_MM_WIDE=0: run wide tiles on the narrow kernel (comparison aid)
    const char* env = std::getenv("PNV_GROUP_MM_WIDE");
    return !(env != nullptr && env[0] == '0');
  }();
  const bool wide = wide_ok && tile_n >= 64 && !trace_enabled();
  static const bool b4d_ok = [] {    // PNV_GROUP_MM_B4D=0: one activation copy per 256-K chunk (comparison aid)
    const char* env = std::getenv("PNV_GROUP_MM_B4D");
    return !(env != nullptr && env[0] == '0');
  }();
  p.b_4d = (b4d_ok && k % 256 == 0 && !trace_enabled()) ? 1 : 0;
  if (p.b_4d) {
    if (int rc = make_map_b4(&map_b, b_act, (uint64_t)k / 2, (uint64_t)max_n, (uint64_t)experts, (uint32_t)tile_n,
                             (uint32_t)stage_k / 256))
      return rc;
  } else if (int rc = make_map(&map_b, b_act, (uint64_t)k / 2, (uint64_t)max_n, (uint64_t)experts, 128,
                               (uint32_t)tile_n, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return rc;
  }

  cudaStream_t s = (cudaStream_t)stream;
  const bool use_pdl = pdl != 0 && pdl_enabled();
  if (wide) {
    switch (tile_n * 1000 + stage_k) {
      case 64256: return launch_wide<64, 256>(map_a, map_b, p, sm_count, use_pdl, s);
      case 64512: return launch_wide<64, 512>(map_a, map_b, p, sm_count, use_pdl, s);
      case 128256: return launch_wide<128, 256>(map_a, map_b, p, sm_count, use_pdl, s);
      case 128512: return launch_wide<128, 512>(map_a, map_b, p, sm_count, use_pdl, s);
      default: return launch_wide<256, 256>(map_a, map_b, p, sm_count, use_pdl, s);
    }
  }
  switch (tile_n * 1000 + stage_k) {
    case 16512: return launch<16, 512, 4>(map_a, map_b, p, sm_count, use_pdl, s);
    case 32512: return launch<32, 512, 4>(map_a, map_b, p, sm_count, use_pdl, s);
    case 64256: return launch<64, 256, 2>(map_a, map_b, p, sm_count, use_pdl, s);
    case 64512: return launch<64, 512, 2>(map_a, map_b, p, sm_count, use_pdl, s);
    case 128256: return launch<128, 256, 1>(map_a, map_b, p, sm_count, use_pdl, s);
    case 128512: return launch<128, 512, 1>(map_a, map_b, p, sm_count, use_pdl, s);
    default: return launch<256, 256, 1>(map_a, map_b, p, sm_count, use_pdl, s);
  }
}

}  // namespace
}  // namespace pnv

extern "C" int pnv_group_mm(void* out, const uint8_t* a_comp, const uint8_t* e_meta, const uint8_t* sfa,
                            const uint8_t* b_act, const uint8_t* sfb, const float* alphas,
                            const int32_t* counts, int experts, int features, int k, int max_n,
                            int config_id, int cluster_m, int cluster_n, int sm_count, int pdl,
                            pnv_stream_t stream) {
  return group_mm_common(out, nullptr, a_comp, e_meta, sfa, b_act, sfb, alphas, counts, experts, features, k,
                         max_n, config_id, cluster_m, cluster_n, sm_count, pdl, stream, nullptr);
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
                                         int sm_count, int pdl, pnv_stream_t stream) {
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
  return group_mm_common(b_out, &f, a_comp, e_meta, sfa, b_act, sfb, alphas, counts, experts, features, k, max_n,
                         fk.base_config, cluster_m, cluster_n, sm_count, pdl, stream, fk.name);
}
