// group_mm: out[e, t, :] = bf16(alpha[e] * W[e] * x[e, t, :]) for t < counts[e], with W stored
// paired-4:8 sparse NVFP4 (a_comp + e_meta + sfa) and x stored NVFP4 (b_act + sfb).
//
// One persistent kernel, one CTA per SM, three warp roles:
//   warp 0 (one lane)  producer: per 256-K stage, two TMA tile loads (compressed weights with the
//                      64-byte swizzle, activations with the 128-byte swizzle; one 3-D tensor map
//                      each covers every expert) and three plain bulk copies (metadata atom, SFA
//                      and SFB scale atoms, which are stored in global memory in exactly the shape
//                      tcgen05.cp consumes, so they need no tensor map);
//   warp 1 (one lane)  MMA issuer: tcgen05.cp of metadata and scales into tensor memory, then two
//                      tcgen05.mma.sp block-scaled instructions (128 x TILE_N x 128 each) per
//                      stage, accumulating in tensor memory; tcgen05.commit releases the stage and,
//                      after the last stage of a tile, publishes the accumulator;
//   warps 2-5          epilogue: tcgen05.ld the accumulator, scale by alpha[e], round to bf16 and
//                      store the rows below the expert's token count.
// Accumulators are double buffered (single buffered for TILE_N = 256, which fills tensor memory),
// so the epilogue of one tile overlaps the main loop of the next.
//
// Tile schedule: every role walks the same list on its own, derived on the device from
// counts[]: experts in order, each contributing ceil(M/128) * ceil(counts[e]/TILE_N) tiles
// (M tile fastest); CTA b takes tiles b, b + grid, ...  No host read of counts, no scheduler
// state in global memory: the launch is fixed-shape and safe to capture in a CUDA graph.
//
// Every mbarrier wait is bounded; a wait that gives up records a code in g_status, and every role
// leaves its loop and meets at the final barrier, where tensor memory is released.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace pnv {
namespace {

__device__ int g_status = 0;

constexpr int kTileM = 128;
constexpr int kStageK = 256;                 // dense K per pipeline stage (two MMA K-blocks)
constexpr int kABytes = kTileM * 64;         // compressed weights: 64 bytes per row per stage
constexpr int kEBytes = 2048;                // one metadata atom
constexpr int kSfaBytes = 1024;              // two scale atoms
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kColE = 448;                   // tensor-memory columns: metadata (4)
constexpr int kColSfa = 456;                 //   weight scales (8)
constexpr int kColSfb = 464;                 //   activation scales (8, or 16 for TILE_N = 256)

enum Status : int {
  kOk = 0, kProducerEmptyTimeout = 1, kMmaFullTimeout = 2, kMmaAccTimeout = 3, kEpilogueTimeout = 4
};

template <int TILE_N>
struct Cfg {
  static constexpr int kBBytes = TILE_N * 128;
  static constexpr int kSfbBytes = TILE_N > 128 ? 2048 : 1024;
  static constexpr int kStageBytes = kABytes + kBBytes + kEBytes + kSfaBytes + kSfbBytes;
  static constexpr int kStages = TILE_N == 256 ? 4 : (TILE_N == 128 ? 7 : 10);
  static_assert(TILE_N == 64 || TILE_N == 128 || TILE_N == 256, "tile widths: 64, 128, 256");
  static constexpr int kAccStages = TILE_N == 256 ? 1 : 2;
  static constexpr int kOffA = 0;
  static constexpr int kOffB = kABytes;
  static constexpr int kOffE = kOffB + kBBytes;
  static constexpr int kOffSfa = kOffE + kEBytes;
  static constexpr int kOffSfb = kOffSfa + kSfaBytes;
  static_assert(kStageBytes % 1024 == 0, "stage buffers must keep 1024-byte alignment");
  static_assert(kAccStages * TILE_N <= kColE, "accumulators overlap the metadata columns");
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
  int k_stages;      // ceil(K / 256)
  int n_kt;          // scale K-atoms per row = MMA K-blocks = ceil(K / 128)
  int e_k_atoms;     // metadata atoms along K = k_stages
  int e_m_atoms;     // metadata atoms along M = n_mt
  int sfb_rt;        // scale row-atoms per expert in sfb = ceil(max_n / 128)
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
    long long local = t - base;
    mt = (int)(local % n_mt);
    nt = (int)(local / n_mt);
    return true;
  }
};

// Traced build (kTrace): every asynchronous operation is issued alone and waited for, each step
// leaves a breadcrumb in host-mapped memory (readable even after a fault killed the context), and
// every copy's addresses and size are checked first; a failed check is recorded and the copy is
// skipped.  Breadcrumb slots per CTA: 0 setup, 1 producer, 2 MMA issuer, 3 epilogue (warp 2),
// 4 first failed check (code), 5..7 its operands.
template <bool kTrace>
__device__ __forceinline__ void crumb(const unsigned* /*unused*/, unsigned* trace, int slot, unsigned code) {
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

template <int TILE_N, bool kTrace>
__global__ void __launch_bounds__(kThreads, 1)
group_mm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const Params p) {
  using C = Cfg<TILE_N>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* acc_full = empty_bar + C::kStages;
  uint64_t* acc_empty = acc_full + C::kAccStages;
  uint64_t* dbg_bar = acc_empty + C::kAccStages;     // two extra barriers, used by the traced build
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dbg_bar + 2);
  int* s_counts = reinterpret_cast<int*>(tmem_slot + 4);
#define CRUMB(slot, code) crumb<kTrace>(nullptr, p.trace, slot, code)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- setup that does not depend on the previous kernel ---------------------------------------
  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    for (int s = 0; s < C::kStages; ++s) { ptx::mbar_init(full_bar + s, 1); ptx::mbar_init(empty_bar + s, 1); }
    for (int a = 0; a < C::kAccStages; ++a) { ptx::mbar_init(acc_full + a, 1); ptx::mbar_init(acc_empty + a, 128); }
    ptx::mbar_init(dbg_bar, 1);
    ptx::mbar_init(dbg_bar + 1, 1);
    ptx::fence_mbar_init();
    CRUMB(0, 1);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
    if (lane == 0) CRUMB(0, 2);
  }
  // counts (and everything else the producer kernels wrote) may only be read after this point
  pdl_wait();
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < p.E; i += kThreads) s_counts[i] = max(0, min(p.counts[i], p.max_n));
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) { CRUMB(0, 3); CRUMB(8, tmem_base); CRUMB(9, ptx::smem_u32(smem)); CRUMB(10, ptx::smem_u32(full_bar)); }

  TileWalk walk;
  walk.init<TILE_N>(s_counts, p.E, p.n_mt);

  if (warp == 0) {
    // =============================== producer ===============================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t dbg_phase = 0;
      (void)dbg_phase;
      bool ok = true;
      for (long long t = blockIdx.x; ok; t += gridDim.x) {
        int mt, nt;
        if (!walk.seek<TILE_N>(t, mt, nt)) break;
        const int e = walk.e;
        const long long e_atom0 = ((long long)e * p.e_k_atoms) * p.e_m_atoms + mt;
        const long long sfa_atom0 = ((long long)e * p.n_mt + mt) * p.n_kt;
        const int n0 = nt * TILE_N;
        const long long sfb_atom0 = ((long long)e * p.sfb_rt + (n0 >> 7)) * p.n_kt;
        const int sfb_row_atoms = TILE_N > 128 ? min(2, p.sfb_rt - (n0 >> 7)) : 1;
        for (int ks = 0; ks < p.k_stages; ++ks) {
          if (!ptx::mbar_wait(empty_bar + stage, phase ^ 1)) {
            atomicExch(&g_status, kProducerEmptyTimeout);
            ok = false;
            break;
          }
          uint8_t* st = stage_base + stage * C::kStageBytes;
          const int k_atoms = min(2, p.n_kt - 2 * ks);         // MMA K-blocks present in this stage
          const uint32_t sf_bytes = 512u * k_atoms;
          const uint32_t tx = kABytes + C::kBBytes + kEBytes + sf_bytes * (1 + sfb_row_atoms);
          const uint8_t* e_src = p.e_meta + (e_atom0 + (long long)ks * p.e_m_atoms) * 2048;
          const uint8_t* sfa_src = p.sfa + (sfa_atom0 + 2 * ks) * 512;
          if (!kTrace) {
            ptx::mbar_arrive_expect_tx(full_bar + stage, tx);
            ptx::tma_load_3d(st + C::kOffA, &map_a, full_bar + stage, ks * 64, mt * kTileM, e);
            ptx::tma_load_3d(st + C::kOffB, &map_b, full_bar + stage, ks * 128, n0, e);
            ptx::bulk_load(st + C::kOffE, e_src, kEBytes, full_bar + stage);
            ptx::bulk_load(st + C::kOffSfa, sfa_src, sf_bytes, full_bar + stage);
            for (int ra = 0; ra < sfb_row_atoms; ++ra)
              ptx::bulk_load(st + C::kOffSfb + ra * 1024,
                             p.sfb + (sfb_atom0 + (long long)ra * p.n_kt + 2 * ks) * 512, sf_bytes,
                             full_bar + stage);
          } else {
            // one copy at a time on a private barrier, then a plain arrive publishes the stage
            uint32_t dphase = dbg_phase;
            auto one = [&](unsigned code, uint32_t bytes, auto issue) {
              CRUMB(1, code);
              ptx::mbar_arrive_expect_tx(dbg_bar, bytes);
              issue();
              bool done = ptx::mbar_wait(dbg_bar, dphase);
              dphase ^= 1;
              CRUMB(1, code + (done ? 1 : 2));
            };
            if (check_copy<kTrace>(p.trace, 100, ptx::smem_u32(st + C::kOffA), 0, kABytes, 1024))
              one(110, kABytes, [&] { ptx::tma_load_3d(st + C::kOffA, &map_a, dbg_bar, ks * 64, mt * kTileM, e); });
            if (check_copy<kTrace>(p.trace, 101, ptx::smem_u32(st + C::kOffB), 0, C::kBBytes, 1024))
              one(120, C::kBBytes, [&] { ptx::tma_load_3d(st + C::kOffB, &map_b, dbg_bar, ks * 128, n0, e); });
            if (check_copy<kTrace>(p.trace, 102, ptx::smem_u32(st + C::kOffE), (uint64_t)e_src, kEBytes, 16))
              one(130, kEBytes, [&] { ptx::bulk_load(st + C::kOffE, e_src, kEBytes, dbg_bar); });
            if (check_copy<kTrace>(p.trace, 103, ptx::smem_u32(st + C::kOffSfa), (uint64_t)sfa_src, sf_bytes, 16))
              one(140, sf_bytes, [&] { ptx::bulk_load(st + C::kOffSfa, sfa_src, sf_bytes, dbg_bar); });
            for (int ra = 0; ra < sfb_row_atoms; ++ra) {
              const uint8_t* sfb_src = p.sfb + (sfb_atom0 + (long long)ra * p.n_kt + 2 * ks) * 512;
              if (check_copy<kTrace>(p.trace, 104, ptx::smem_u32(st + C::kOffSfb + ra * 1024), (uint64_t)sfb_src,
                                     sf_bytes, 16))
                one(150, sf_bytes, [&] { ptx::bulk_load(st + C::kOffSfb + ra * 1024, sfb_src, sf_bytes, dbg_bar); });
            }
            dbg_phase = dphase;
            ptx::mbar_arrive(full_bar + stage);
            CRUMB(1, 160);
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // give copies already in flight time to land before the CTA's shared memory is released
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::mma_sp_nvf4_idesc(TILE_N);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0, mma_dbg_phase = 0;
      (void)mma_dbg_phase;
      bool ok = true;
      for (long long t = blockIdx.x; ok; t += gridDim.x) {
        int mt, nt;
        if (!walk.seek<TILE_N>(t, mt, nt)) break;
        if (!ptx::mbar_wait(acc_empty + acc, acc_phase ^ 1)) {
          atomicExch(&g_status, kMmaAccTimeout);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TILE_N;
        // The scales of a 64-wide tile's rows sit 0 or 2 columns into the 128-row atom.  The MMA
        // faults (misaligned address) on an odd column offset, which is why there is no 32-wide tile.
        const uint32_t sfb_col = tmem_base + kColSfb + (TILE_N < 128 ? ((nt * TILE_N) & 127) >> 5 : 0);
        for (int ks = 0; ks < p.k_stages; ++ks) {
          if (!ptx::mbar_wait(full_bar + stage, phase)) {
            atomicExch(&g_status, kMmaFullTimeout);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t st = ptx::smem_u32(stage_base + stage * C::kStageBytes);
          const int k_atoms = min(2, p.n_kt - 2 * ks);
          auto settle = [&](unsigned code) {   // traced build: wait until the operation just issued retires
            if (kTrace) {
              CRUMB(2, code);
              ptx::tc_commit(dbg_bar + 1);
              bool done = ptx::mbar_wait(dbg_bar + 1, mma_dbg_phase);
              mma_dbg_phase ^= 1;
              CRUMB(2, code + (done ? 1 : 2));
            }
          };
          if (kTrace) CRUMB(2, 200);
          ptx::tc_cp_128x128b(tmem_base + kColE, ptx::smem_desc(st + C::kOffE, 128, 0, 0));
          settle(210);
          for (int ka = 0; ka < k_atoms; ++ka) {
            ptx::tc_cp_32x128b_warpx4(tmem_base + kColSfa + ka * 4,
                                      ptx::smem_desc(st + C::kOffSfa + ka * 512, 128, 0, 0));
            if (TILE_N > 128) {
              ptx::tc_cp_32x128b_warpx4(tmem_base + kColSfb + ka * 8,
                                        ptx::smem_desc(st + C::kOffSfb + ka * 512, 128, 0, 0));
              ptx::tc_cp_32x128b_warpx4(tmem_base + kColSfb + ka * 8 + 4,
                                        ptx::smem_desc(st + C::kOffSfb + 1024 + ka * 512, 128, 0, 0));
            } else {
              ptx::tc_cp_32x128b_warpx4(tmem_base + kColSfb + ka * 4,
                                        ptx::smem_desc(st + C::kOffSfb + ka * 512, 128, 0, 0));
            }
            settle(220 + 10 * ka);
          }
          for (int ka = 0; ka < k_atoms; ++ka) {
            const uint64_t a_desc = ptx::smem_desc(st + C::kOffA + ka * 32, 512, 16, 4);
            const uint64_t b_desc = ptx::smem_desc(st + C::kOffB + ka * 64, 1024, 16, 2);
            ptx::tc_mma_sp_nvf4(d_tmem, a_desc, b_desc, idesc, (ks | ka) != 0 ? 1u : 0u,
                                tmem_base + kColSfa + ka * 4,
                                sfb_col + ka * (TILE_N > 128 ? 8 : 4), tmem_base + kColE + ka * 2);
            settle(240 + 10 * ka);
          }
          ptx::tc_commit(empty_bar + stage);   // stage reusable once these MMAs and copies retire
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        ptx::tc_commit(acc_full + acc);        // accumulator complete
        if (kTrace) CRUMB(2, 290);
        if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // =============================== epilogue ===============================
    const int sub = warp & 3;                  // tensor-memory lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (long long t = blockIdx.x;; t += gridDim.x) {
      int mt, nt;
      if (!walk.seek<TILE_N>(t, mt, nt)) break;
      const int e = walk.e;
      const int cnt = s_counts[e];
      if (!ptx::mbar_wait(acc_full + acc, acc_phase)) {
        atomicExch(&g_status, kEpilogueTimeout);
        break;
      }
      ptx::tc_fence_after();
      if (kTrace && threadIdx.x == 64) CRUMB(3, 300);
      const float alpha = p.alphas[e];
      const int m = mt * kTileM + sub * 32 + lane;
      const int n0 = nt * TILE_N;
      __nv_bfloat16* out_e = p.out + (long long)e * p.max_n * p.M;
#pragma unroll 1
      for (int c0 = 0; c0 < TILE_N; c0 += 32) {
        if (n0 + c0 >= cnt) break;             // warp-uniform
        uint32_t r[32];
        ptx::tc_ld_32x32(tmem_base + ((uint32_t)(sub * 32) << 16) + acc * TILE_N + c0, r);
        ptx::tc_ld_wait();
        if (kTrace && threadIdx.x == 64) CRUMB(3, 310);
        if (m < p.M) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int n = n0 + c0 + i;
            if (n < cnt)
              out_e[(long long)n * p.M + m] = __float2bfloat16_rn(__fmul_rn(alpha, __uint_as_float(r[i])));
          }
        }
      }
      if (kTrace && threadIdx.x == 64) CRUMB(3, 320);
      ptx::tc_fence_before();
      ptx::mbar_arrive(acc_empty + acc);
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
    if (lane == 0) CRUMB(0, 9);
  }
#undef CRUMB
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

bool trace_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* env = std::getenv("PNV_GROUP_MM_TRACE");
    v = (env != nullptr && env[0] == '1') ? 1 : 0;
  }
  return v == 1;
}

template <int TILE_N, bool kTrace>
int launch_impl(const CUtensorMap& map_a, const CUtensorMap& map_b, const Params& p, int sm_count, bool pdl,
                cudaStream_t stream) {
  using C = Cfg<TILE_N>;
  const size_t smem = 1024 + (size_t)C::kStages * C::kStageBytes + 8 * (2 * C::kStages + 2 * C::kAccStages + 2) +
                      16 + 4 * (size_t)p.E;
  PNV_REQUIRE(smem <= 227 * 1024, "group_mm: %d experts need %zu bytes of shared memory (limit 232448)", p.E,
              smem);
  // opt in to the large dynamic shared-memory carve-out once per device
  static bool opted_in[64] = {};
  int dev = 0;
  PNV_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !opted_in[dev]) {
    PNV_CUDA(cudaFuncSetAttribute(group_mm_kernel<TILE_N, kTrace>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  227 * 1024));
    if (dev >= 0 && dev < 64) opted_in[dev] = true;
  }
  long long max_tiles = (long long)p.E * p.n_mt * ceil_div_i(p.max_n, TILE_N);
  int grid = (int)(max_tiles < sm_count ? max_tiles : sm_count);
  if (grid < 1) grid = 1;
  PNV_CUDA(launch_pdl(group_mm_kernel<TILE_N, kTrace>, dim3(grid), dim3(kThreads), smem, stream, pdl, map_a,
                      map_b, p));
  return PNV_OK;
}

template <int TILE_N>
int launch(const CUtensorMap& map_a, const CUtensorMap& map_b, Params& p, int sm_count, bool pdl,
           cudaStream_t stream) {
  if (!trace_enabled()) {
    p.trace = nullptr;
    return launch_impl<TILE_N, false>(map_a, map_b, p, sm_count, pdl, stream);
  }
  if (g_trace_host == nullptr) {
    PNV_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&g_trace_host), kTraceWords * sizeof(unsigned),
                           cudaHostAllocMapped));
    PNV_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&g_trace_dev), g_trace_host, 0));
  }
  for (int i = 0; i < kTraceWords; ++i) g_trace_host[i] = 0;
  p.trace = g_trace_dev;
  return launch_impl<TILE_N, true>(map_a, map_b, p, sm_count, false, stream);
}

struct Kind { const char* name; bool two_sm; int tile_n; };
const Kind kKinds[] = {
    {"sparse_2sm_256x128", true, 128},   {"sparse_2sm_256x256", true, 256},
    {"sparse_1sm_128x128", false, 128},  {"sparse_1sm_128x256", false, 256},
    {"sparse_2sm_256x64", true, 64},     {"sparse_1sm_128x64", false, 64},
    {"sparse_2sm_256x64_k512", true, 64}, {"sparse_1sm_128x64_k512", false, 64},
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

extern "C" int pnv_group_mm_debug_trace(unsigned* words_out, int n_words) {
  PNV_REQUIRE(words_out && n_words >= 0, "bad trace buffer");
  for (int i = 0; i < n_words; ++i)
    words_out[i] = (g_trace_host != nullptr && i < kTraceWords) ? ((volatile unsigned*)g_trace_host)[i] : 0u;
  return PNV_OK;
}

extern "C" int pnv_group_mm(void* out, const uint8_t* a_comp, const uint8_t* e_meta, const uint8_t* sfa,
                            const uint8_t* b_act, const uint8_t* sfb, const float* alphas,
                            const int32_t* counts, int experts, int features, int k, int max_n,
                            int config_id, int cluster_m, int cluster_n, int sm_count, int pdl,
                            pnv_stream_t stream) {
  PNV_REQUIRE(out && a_comp && e_meta && sfa && b_act && sfb && alphas && counts, "null pointer argument");
  PNV_REQUIRE(experts >= 1 && features >= 1 && max_n >= 1, "experts, features and max_n must be positive");
  PNV_REQUIRE(k > 0 && k % kSfBlock == 0, "K must be a multiple of %d, got %d", kSfBlock, k);
  PNV_REQUIRE(config_id >= 0 && config_id < kNumKinds, "config_id must be in [0, %d), got %d", kNumKinds,
              config_id);
  const Kind& kind = kKinds[config_id];
  auto pow2_le4 = [](int x) { return x == 1 || x == 2 || x == 4; };
  PNV_REQUIRE(pow2_le4(cluster_m) && pow2_le4(cluster_n) && cluster_m * cluster_n <= 16,
              "%s: cluster dims must be powers of two <= 4 with product <= 16, got %dx%d", kind.name,
              cluster_m, cluster_n);
  PNV_REQUIRE(!kind.two_sm || cluster_m % 2 == 0,
              "%s is a 2SM kernel and needs an even cluster_m, got %d", kind.name, cluster_m);
  PNV_REQUIRE((reinterpret_cast<uintptr_t>(a_comp) | reinterpret_cast<uintptr_t>(b_act) |
               reinterpret_cast<uintptr_t>(e_meta) | reinterpret_cast<uintptr_t>(sfa) |
               reinterpret_cast<uintptr_t>(sfb)) % 16 == 0,
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
  p.E = experts; p.M = features; p.K = k; p.max_n = max_n;
  p.n_mt = ceil_div_i(features, kTileM);
  p.k_stages = ceil_div_i(k, kStageK);
  p.n_kt = sf_k_atoms(k);
  p.e_k_atoms = wd.k_e / 16;
  p.e_m_atoms = wd.m_e / 128;
  p.sfb_rt = sf_row_atoms(max_n);

  CUtensorMap map_a, map_b;
  if (int rc = make_map(&map_a, a_comp, (uint64_t)wd.k_ac / 2, (uint64_t)wd.m_ac, (uint64_t)experts, 64,
                        kTileM, CU_TENSOR_MAP_SWIZZLE_64B))
    return rc;
  if (int rc = make_map(&map_b, b_act, (uint64_t)k / 2, (uint64_t)max_n, (uint64_t)experts, 128,
                        (uint32_t)kind.tile_n, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;

  cudaStream_t s = (cudaStream_t)stream;
  const bool use_pdl = pdl != 0 && pdl_enabled();
  switch (kind.tile_n) {
    case 64: return launch<64>(map_a, map_b, p, sm_count, use_pdl, s);
    case 128: return launch<128>(map_a, map_b, p, sm_count, use_pdl, s);
    default: return launch<256>(map_a, map_b, p, sm_count, use_pdl, s);
  }
}
