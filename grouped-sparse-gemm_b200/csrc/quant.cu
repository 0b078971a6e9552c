// Activation quantizers: bf16 -> e2m1 codes + one UE4M3 scale per 32 elements, written straight
// into the grouped GEMM's B-operand layouts (row-major codes, swizzled scale atoms).
//
// quant_act and silu_mul_quant_act walk the *scale buffer*: one warp owns one 16-byte line of a
// scale atom, i.e. the 4 rows {r, r+32, r+64, r+96} x 4 K-blocks whose scales share that line.
// The warp quantizes the (up to) 4 x 128 elements behind it with 128-bit loads, reduces each
// block's amax with one shuffle, and writes the line once -- quantized scales where a row is live,
// the benign byte 0x38 everywhere else -- so the scale buffer is fully defined without a separate
// fill pass and without byte-sized stores.  Lines whose rows are all past the expert's token
// count cost one 16-byte store.
//
// scatter_quant_act is driven by a routing list instead (source token -> destination row), so its
// scale buffer is pre-filled with a memset node and each warp quantizes 256 elements of one routed
// row.
#include <mutex>

#include "common.cuh"

namespace pnv {
namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerBlock = kThreads / 32;

// Gather the 16 scale bytes of a line from the lanes that own them (lane g*8 + 2*kq holds the
// byte of row group g, K-block kq) and store them as four 32-bit words.
__device__ __forceinline__ void store_sf_line(uint8_t* line, uint32_t my_byte, int lane) {
  int g8 = lane & ~7;
  uint32_t w = __shfl_sync(0xffffffffu, my_byte, g8 + 0) |
               (__shfl_sync(0xffffffffu, my_byte, g8 + 2) << 8) |
               (__shfl_sync(0xffffffffu, my_byte, g8 + 4) << 16) |
               (__shfl_sync(0xffffffffu, my_byte, g8 + 6) << 24);
  if ((lane & 7) == 0) *reinterpret_cast<uint32_t*>(line + (lane >> 3) * 4) = w;
}

// Where a live row's values come from.
//   kPlain   x is [E, max_n, K]
//   kGated   x is [E, max_n, 2K] holding gate and up; the gated activation is applied first
enum LineSource : int { kPlain = 0, kGated = 1 };

template <int kSrc>
__global__ void __launch_bounds__(kThreads)
quant_lines_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gscale,
                   int gscale_per_expert, const int* __restrict__ counts, int E, int max_n, int K,
                   int interleaved, GatedAct act, uint8_t* __restrict__ b_act,
                   uint8_t* __restrict__ sfb) {
  pdl_wait();
  pdl_launch_dependents();
  const int KB = K / kSfBlock;
  const int n_rt = sf_row_atoms(max_n);
  const int n_kt = sf_k_atoms(K);
  // line arithmetic in 32 bits (the host checks the line count): 64-bit divisions per line once
  // cost more instructions than the quantization itself
  const unsigned lines = (unsigned)E * n_rt * n_kt * 32u;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 3;          // row group inside the atom: rows rr + 32 g
  const int j = lane & 7;           // 16-element piece of the 128-element segment
  const unsigned warp0 = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const unsigned nwarps = gridDim.x * kWarpsPerBlock;
  const uint32_t benign4 = kBenignSf * 0x01010101u;

  for (unsigned c = warp0; c < lines; c += nwarps) {
    const int rr = (int)(c & 31);
    const unsigned a = c >> 5;
    const unsigned a_kt = a / (unsigned)n_kt;
    const int kt = (int)(a - a_kt * n_kt);
    const int e = (int)(a_kt / (unsigned)n_rt);
    const int rt = (int)(a_kt - (unsigned)e * n_rt);
    const int cnt = min(counts[e], max_n);
    uint8_t* line = sfb + (long long)c * 16;
    if (rt * 128 + rr >= cnt) {   // no live row behind this line
      if (lane == 0) *reinterpret_cast<uint4*>(line) = make_uint4(benign4, benign4, benign4, benign4);
      continue;
    }
    const int r = rt * 128 + rr + 32 * g;
    const int kb = kt * 4 + (j >> 1);
    const bool live = (r < cnt) && (kb < KB);
    const int k0 = kb * kSfBlock + (j & 1) * 16;
    uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
    float f0[8], f1[8];
    if (live) {
      const long long row = (long long)e * max_n + r;
      if (kSrc == kPlain) {
        const uint4* p = reinterpret_cast<const uint4*>(x + row * K + k0);
        v0 = __ldg(p);
        v1 = __ldg(p + 1);
        unpack8(v0, f0);
        unpack8(v1, f1);
      } else {
        const __nv_bfloat16* base = x + row * (2LL * K);
        const int gate_off = interleaved ? kb * 64 + (j & 1) * 16 : k0;
        const int up_off = interleaved ? gate_off + 32 : K + k0;
        const uint4* pg = reinterpret_cast<const uint4*>(base + gate_off);
        const uint4* pu = reinterpret_cast<const uint4*>(base + up_off);
        uint4 g0 = __ldg(pg), g1 = __ldg(pg + 1), u0 = __ldg(pu), u1 = __ldg(pu + 1);
        float ga[8], ua[8];
        unpack8(g0, ga); unpack8(u0, ua);
        float gb[8], ub[8];
        unpack8(g1, gb); unpack8(u1, ub);
        if (act.kind == PNV_ACT_SILU && act.silu_tab != nullptr) {   // straight-line: 16 independent lookups
#pragma unroll
          for (int i = 0; i < 8; ++i) { f0[i] = silu_mul(ga[i], ua[i], act.silu_tab); f1[i] = silu_mul(gb[i], ub[i], act.silu_tab); }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) f0[i] = gated_act(ga[i], ua[i], act);
#pragma unroll
          for (int i = 0; i < 8; ++i) f1[i] = gated_act(gb[i], ub[i], act);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) { f0[i] = 0.f; f1[i] = 0.f; }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fmaxf(fabsf(f0[i]), fabsf(f1[i])));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    uint32_t sf_byte = kBenignSf;
    if (live) {
      const float gs = gscale_per_expert ? gscale[e] : gscale[0];
      float inv;
      block_scale(amax, gs, sf_byte, inv);
      uint2 codes = make_uint2(quant8(f0, inv), quant8(f1, inv));
      const long long row = (long long)e * max_n + r;
      *reinterpret_cast<uint2*>(b_act + row * (K / 2) + k0 / 2) = codes;
    }
    store_sf_line(line, sf_byte, lane);
  }
}

// Four adjacent lanes hold the scale bytes of four consecutive K-blocks; lane 4j returns their word.
__device__ __forceinline__ uint32_t gather_sf_word(uint32_t my_byte) {
  return my_byte | (__shfl_down_sync(0xffffffffu, my_byte, 1) << 8) |
         (__shfl_down_sync(0xffffffffu, my_byte, 2) << 16) | (__shfl_down_sync(0xffffffffu, my_byte, 3) << 24);
}

// One 32-element block in one lane: 64 bytes in, amax, scale, 16 bytes of codes.  Doing the whole
// block in a lane runs the scale step (two IEEE divisions, two format conversions) once per block
// instead of once per 8 elements, which is what bounds these kernels on B200.
struct BlockRegs {
  float f[4][8];
};
__device__ __forceinline__ void load_block(const uint4* src, BlockRegs& b) {
  uint4 v0 = __ldg(src), v1 = __ldg(src + 1), v2 = __ldg(src + 2), v3 = __ldg(src + 3);
  unpack8(v0, b.f[0]); unpack8(v1, b.f[1]); unpack8(v2, b.f[2]); unpack8(v3, b.f[3]);
}
__device__ __forceinline__ float block_amax(const BlockRegs& b) {
  float m = 0.f;
#pragma unroll
  for (int q = 0; q < 4; ++q)
#pragma unroll
    for (int z = 0; z < 8; ++z) m = fmaxf(m, fabsf(b.f[q][z]));
  return m;
}
__device__ __forceinline__ uint4 block_codes(const BlockRegs& b, float inv) {
  return make_uint4(quant8(b.f[0], inv), quant8(b.f[1], inv), quant8(b.f[2], inv), quant8(b.f[3], inv));
}

// One routed row by one warp: 32 K-blocks (1024 elements) at a time, one block per lane; a row's four scales
// of one 128-K group are one aligned word of the swizzled layout.  `w` is the (already bf16-rounded) router
// weight when `weighted`.
__device__ __forceinline__ void quantize_routed_row(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                    uint8_t* __restrict__ sf_row, int KB, float gs, bool weighted,
                                                    float w, int lane) {
  for (int kb0 = 0; kb0 < KB; kb0 += 32) {
    const int kb = kb0 + lane;
    uint32_t sf_byte = kBenignSf;   // blocks past K keep the benign byte in the layout's slop
    if (kb < KB) {
      BlockRegs b;
      load_block(src + kb * 4, b);
      if (weighted) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int z = 0; z < 8; ++z) b.f[q][z] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(b.f[q][z], w)));
      }
      float inv;
      block_scale(block_amax(b), gs, sf_byte, inv);
      dst[kb] = block_codes(b, inv);
    }
    const uint32_t word = gather_sf_word(sf_byte);
    if ((lane & 3) == 0 && kb < KB) *reinterpret_cast<uint32_t*>(sf_row + (kb >> 2) * 512) = word;
  }
}

// scatter_quant_act: one warp per routing of the flat plan.
__global__ void __launch_bounds__(kThreads)
scatter_quant_kernel(const __nv_bfloat16* __restrict__ a1, const long long* __restrict__ flat_tok,
                     const long long* __restrict__ dest_global, const float* __restrict__ topk_w,
                     const float* __restrict__ gscale, int gscale_per_expert, unsigned n_routes,
                     int K, int E, int cap, uint8_t* __restrict__ b_act, uint8_t* __restrict__ sfb) {
  pdl_wait();
  pdl_launch_dependents();
  const int KB = K / kSfBlock;
  const int n_rt = sf_row_atoms(cap);
  const int n_kt = sf_k_atoms(K);
  const long long trash = (long long)E * cap;
  const int lane = threadIdx.x & 31;
  const unsigned warp0 = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const unsigned nwarps = gridDim.x * kWarpsPerBlock;
  for (unsigned i = warp0; i < n_routes; i += nwarps) {
    const long long dest = dest_global[i];
    if (dest == trash) continue;   // dropped routing: non-local expert or past capacity
    const int e = (int)((unsigned)dest / (unsigned)cap);     // dest < E * cap < 2^31
    const int r = (int)dest - e * cap;
    const float gs = gscale_per_expert ? gscale[e] : gscale[0];
    const bool weighted = topk_w != nullptr;
    const float w = weighted ? __bfloat162float(__float2bfloat16_rn(topk_w[i])) : 1.f;
    quantize_routed_row(reinterpret_cast<const uint4*>(a1 + flat_tok[i] * K),
                        reinterpret_cast<uint4*>(b_act + dest * (K / 2)), sfb + sf_offset(e, r, 0, n_rt, n_kt), KB, gs,
                        weighted, w, lane);
  }
}

// scatter_quant_act_planned: one warp per row slot (e, r) of the batched operand; slots at or past counts[e] are
// skipped (their scales keep the benign fill laid down before the launch).
__global__ void __launch_bounds__(kThreads)
scatter_planned_rows_kernel(const __nv_bfloat16* __restrict__ a1, const int* __restrict__ src_tok,
                            const int* __restrict__ src_route, const float* __restrict__ topk_w,
                            const float* __restrict__ gscale, int gscale_per_expert, const int* __restrict__ counts,
                            int K, int E, int cap, uint8_t* __restrict__ b_act, uint8_t* __restrict__ sfb) {
  pdl_wait();
  pdl_launch_dependents();
  const int KB = K / kSfBlock;
  const int n_rt = sf_row_atoms(cap);
  const int n_kt = sf_k_atoms(K);
  const int lane = threadIdx.x & 31;
  const unsigned slots = (unsigned)E * (unsigned)cap;
  const unsigned warp0 = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const unsigned nwarps = gridDim.x * kWarpsPerBlock;
  for (unsigned slot = warp0; slot < slots; slot += nwarps) {
    const int e = (int)(slot / (unsigned)cap);
    const int r = (int)(slot - (unsigned)e * (unsigned)cap);
    if (r >= min(counts[e], cap)) {
      // jump to the next expert's first slot that this warp owns
      const unsigned next = (unsigned)(e + 1) * (unsigned)cap;
      const unsigned skip = (next - slot + nwarps - 1) / nwarps;
      slot += (skip - 1) * nwarps;
      continue;
    }
    const float gs = gscale_per_expert ? gscale[e] : gscale[0];
    const bool weighted = topk_w != nullptr;
    const float w = weighted ? __bfloat162float(__float2bfloat16_rn(topk_w[src_route[slot]])) : 1.f;
    quantize_routed_row(reinterpret_cast<const uint4*>(a1 + (long long)src_tok[slot] * K),
                        reinterpret_cast<uint4*>(b_act + (long long)slot * (K / 2)), sfb + sf_offset(e, r, 0, n_rt, n_kt),
                        KB, gs, weighted, w, lane);
  }
}

// scatter_fp4_planned / scatter_fp4_wire: already quantized rows into the batched operands, one warp per row slot.
// Codes are copied 16 bytes per lane; the row's scales go from natural order into the swizzled layout four
// K-blocks (one aligned word of both layouts) at a time.  Slots at or past counts[e] are skipped; their scales
// keep the benign fill laid down before the launch.
__global__ void __launch_bounds__(kThreads)
scatter_fp4_rows_kernel(const uint8_t* __restrict__ q, long long q_pitch, const uint8_t* __restrict__ q_sf,
                        long long sf_pitch, const int* __restrict__ src_tok, const int* __restrict__ counts, int K, int E,
                        int cap, uint8_t* __restrict__ b_act, uint8_t* __restrict__ sfb) {
  pdl_wait();
  pdl_launch_dependents();
  const int KB = K / kSfBlock;
  const int n_rt = sf_row_atoms(cap);
  const int n_kt = sf_k_atoms(K);
  const int lane = threadIdx.x & 31;
  const unsigned slots = (unsigned)E * (unsigned)cap;
  const unsigned warp0 = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const unsigned nwarps = gridDim.x * kWarpsPerBlock;
  const bool words = (KB % 4) == 0 && (sf_pitch % 4) == 0 && (reinterpret_cast<uintptr_t>(q_sf) % 4) == 0;
  for (unsigned slot = warp0; slot < slots; slot += nwarps) {
    const int e = (int)(slot / (unsigned)cap);
    const int r = (int)(slot - (unsigned)e * (unsigned)cap);
    if (r >= min(counts[e], cap)) {
      const unsigned next = (unsigned)(e + 1) * (unsigned)cap;       // on to the next expert's first slot of this warp
      slot += ((next - slot + nwarps - 1) / nwarps - 1) * nwarps;
      continue;
    }
    const long long t = src_tok[slot];
    const uint4* src = reinterpret_cast<const uint4*>(q + t * q_pitch);
    uint4* dst = reinterpret_cast<uint4*>(b_act + (long long)slot * (K / 2));
    for (int v = lane; v < K / 32; v += 32) dst[v] = __ldg(src + v);
    const uint8_t* sf_src = q_sf + t * sf_pitch;
    uint8_t* sf_row = sfb + sf_offset(e, r, 0, n_rt, n_kt);        // K-block kb of this row: + (kb >> 2) * 512 + (kb & 3)
    if (words) {
      for (int w = lane; w < KB / 4; w += 32)
        *reinterpret_cast<uint32_t*>(sf_row + w * 512) = __ldg(reinterpret_cast<const uint32_t*>(sf_src) + w);
    } else {
      for (int kb = lane; kb < KB; kb += 32) sf_row[(kb >> 2) * 512 + (kb & 3)] = __ldg(sf_src + kb);
    }
  }
}

// quant_rows: token-order rows -> row-major codes and natural-order scales, one shared global scale.
// One warp per row, one 32-element block per lane; four scales leave as one word.
__global__ void __launch_bounds__(kThreads)
quant_rows_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gscale, unsigned T, int K,
                  uint8_t* __restrict__ q, uint8_t* __restrict__ q_sf) {
  pdl_wait();
  pdl_launch_dependents();
  const int KB = K / kSfBlock;
  const int lane = threadIdx.x & 31;
  const float gs = gscale[0];
  const unsigned warp0 = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const unsigned nwarps = gridDim.x * kWarpsPerBlock;
  const bool sf_words = (KB % 4) == 0;     // rows of scales are then 4-byte aligned
  for (unsigned t = warp0; t < T; t += nwarps) {
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * K);
    uint4* dst = reinterpret_cast<uint4*>(q + (long long)t * (K / 2));
    uint8_t* sf_row = q_sf + (long long)t * KB;
    for (int kb0 = 0; kb0 < KB; kb0 += 32) {
      const int kb = kb0 + lane;
      uint32_t sf_byte = 0;
      if (kb < KB) {
        BlockRegs b;
        load_block(src + kb * 4, b);
        float inv;
        block_scale(block_amax(b), gs, sf_byte, inv);
        dst[kb] = block_codes(b, inv);
        if (!sf_words) sf_row[kb] = (uint8_t)sf_byte;
      }
      const uint32_t word = gather_sf_word(sf_byte);
      if (sf_words && (lane & 3) == 0 && kb < KB) *reinterpret_cast<uint32_t*>(sf_row + kb) = word;
    }
  }
}

__global__ void __launch_bounds__(kThreads)
gated_act_kernel(const __nv_bfloat16* __restrict__ x2, long long rows, int N, int interleaved,
                 GatedAct act, __nv_bfloat16* __restrict__ y) {
  const int per_row = N / 8;
  const long long total = rows * per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long row = idx / per_row;
    const int k0 = (int)(idx - row * per_row) * 8;
    const __nv_bfloat16* base = x2 + row * (2LL * N);
    const int gate_off = interleaved ? (k0 / 32) * 64 + (k0 % 32) : k0;
    const int up_off = interleaved ? gate_off + 32 : N + k0;
    uint4 gv = __ldg(reinterpret_cast<const uint4*>(base + gate_off));
    uint4 uv = __ldg(reinterpret_cast<const uint4*>(base + up_off));
    float ga[8], ua[8];
    unpack8(gv, ga);
    unpack8(uv, ua);
    __nv_bfloat16 o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16_rn(gated_act(ga[i], ua[i], act));
    *reinterpret_cast<uint4*>(y + row * N + k0) = *reinterpret_cast<const uint4*>(o);
  }
}

// Wire rows of the expert-parallel dispatch: one routed token row as it crosses the link,
//   [K/2 bytes of e2m1 codes][K/32 UE4M3 scales][padding to 16 bytes][int32 expert id local to the receiver][12 bytes]
// in fixed-capacity slabs of `slab` rows per destination rank.  Slot s of slab w is live when
// s < slab_counts[w]; a dead slot only gets its expert id, -1, which the receiver's dispatch_plan
// treats like any routing that is not for one of its experts.
__host__ __device__ inline long long wire_row_bytes(int K) { return (long long)round_up_i(K / 2 + K / kSfBlock, 16) + 16; }

template <class IdT>
__global__ void __launch_bounds__(128)
pack_wire_rows_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ q_sf, const IdT* __restrict__ ids,
                      const int* __restrict__ slot_tok, const int* __restrict__ slot_route,
                      const int* __restrict__ slab_counts, int slab, int experts_per_rank, int K,
                      uint8_t* __restrict__ wire, const RowParts parts) {
  pdl_wait();
  pdl_launch_dependents();
  const long long slot = blockIdx.x;
  const int w = (int)(slot / slab);
  const int s = (int)(slot - (long long)w * slab);
  const long long row_bytes = wire_row_bytes(K);
  // (with parts: slab w goes to buffer w, which may be the receiving rank's own memory)
  uint8_t* row = parts.n ? static_cast<uint8_t*>(parts.base[w]) + s * row_bytes : wire + slot * row_bytes;
  int* id_out = reinterpret_cast<int*>(row + row_bytes - 16);
  if (s >= min(slab_counts[w], slab)) {
    if (threadIdx.x == 0) *id_out = -1;
    return;
  }
  const long long t = slot_tok[slot];
  const int code_vecs = K / 32;                       // 16-byte words of codes
  const uint4* src = reinterpret_cast<const uint4*>(q + t * (K / 2));
  uint4* dst = reinterpret_cast<uint4*>(row);
  for (int v = threadIdx.x; v < code_vecs; v += 128) dst[v] = __ldg(src + v);
  const int KB = K / kSfBlock;
  const uint8_t* sf_src = q_sf + t * KB;
  uint8_t* sf_dst = row + K / 2;
  if (KB % 16 == 0) {
    for (int v = threadIdx.x; v < KB / 16; v += 128)
      reinterpret_cast<uint4*>(sf_dst)[v] = __ldg(reinterpret_cast<const uint4*>(sf_src) + v);
  } else {
    for (int b = threadIdx.x; b < KB; b += 128) sf_dst[b] = __ldg(sf_src + b);
  }
  if (threadIdx.x == 0) *id_out = (int)((long long)ids[slot_route[slot]] - (long long)w * experts_per_rank);
}

int grid_for(long long warp_items, int sm_count) {
  long long blocks = (warp_items + kWarpsPerBlock - 1) / kWarpsPerBlock;
  long long cap = (long long)(sm_count > 0 ? sm_count : 148) * 8;   // 8 x 256 threads fill an SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

int check_common(const void* x, const float* gscale, const int32_t* counts, int E, int rows, int K,
                 const uint8_t* b_act, const uint8_t* sfb, const char* kname) {
  PNV_REQUIRE(x && gscale && counts && b_act && sfb, "null pointer argument");
  PNV_REQUIRE(E >= 1 && rows >= 1, "experts and row capacity must be positive, got %d and %d", E, rows);
  PNV_REQUIRE(K > 0 && K % kSfBlock == 0, "%s must be a multiple of %d, got %d", kname, kSfBlock, K);
  PNV_REQUIRE(sf_numel(rows, K, E) / 16 < (1LL << 31) - (1LL << 24), "the scale layout has too many lines for one launch");
  PNV_REQUIRE(sf_numel(rows, K, E) / 16 < (1LL << 40), "scale buffer too large");
  return PNV_OK;
}

}  // namespace

// ---- SiLU table ---------------------------------------------------------------------------------
// 128 KiB inside the library, one copy per device, filled on first use by a kernel on the caller's
// stream; later callers on other streams wait for that kernel through an event (no host wait).  A
// first use inside a stream capture puts the fill kernel into the capture instead (it is
// idempotent), so a graph never depends on work outside it.
static __device__ uint16_t g_silu_tab[65536];
bool g_silu_table_on = true;

__global__ void silu_table_kernel(uint16_t* tab) {
  const unsigned bits = blockIdx.x * blockDim.x + threadIdx.x;
  if (bits < 65536u) tab[bits] = (uint16_t)(__float_as_uint(silu_direct(__uint_as_float(bits << 16))) >> 16);
}

int silu_table(cudaStream_t stream, const uint16_t** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int state[kMaxDevices] = {};          // 0 nothing yet, 1 fill launched, 2 fill known complete
  static uint16_t* ptr[kMaxDevices] = {};
  static cudaEvent_t filled[kMaxDevices] = {};
  int dev = 0;
  PNV_CUDA(cudaGetDevice(&dev));
  PNV_REQUIRE(dev >= 0 && dev < kMaxDevices, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (ptr[dev] == nullptr) {
    void* sym = nullptr;
    PNV_CUDA(cudaGetSymbolAddress(&sym, g_silu_tab));
    ptr[dev] = static_cast<uint16_t*>(sym);
  }
  *out = ptr[dev];
  if (state[dev] == 2) return PNV_OK;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  PNV_CUDA(cudaStreamIsCapturing(stream, &cap));
  const bool capturing = cap != cudaStreamCaptureStatusNone;
  if (state[dev] == 1 && !capturing) {
    cudaError_t q = cudaEventQuery(filled[dev]);
    if (q == cudaSuccess) { state[dev] = 2; return PNV_OK; }
    if (q != cudaErrorNotReady) return fail(PNV_ERR_CUDA, "cudaEventQuery failed: %s", cudaGetErrorString(q));
    PNV_CUDA(cudaStreamWaitEvent(stream, filled[dev], 0));
    return PNV_OK;
  }
  silu_table_kernel<<<256, 256, 0, stream>>>(ptr[dev]);
  PNV_CUDA(cudaGetLastError());
  if (!capturing && state[dev] == 0) {
    PNV_CUDA(cudaEventCreateWithFlags(&filled[dev], cudaEventDisableTiming));
    PNV_CUDA(cudaEventRecord(filled[dev], stream));
    state[dev] = 1;
  }
  return PNV_OK;
}

int make_gated_act(int act_kind, float beta, float linear_beta, cudaStream_t stream, GatedAct& out) {
  if (act_kind == PNV_ACT_SILU) {
    out = GatedAct{PNV_ACT_SILU, 1.0f, -1.0f, nullptr};
    if (g_silu_table_on)
      if (int rc = silu_table(stream, &out.silu_tab)) return rc;
  } else if (act_kind == PNV_ACT_SITU) {
    PNV_REQUIRE(beta > 0, "situ: beta must be positive, got %g", (double)beta);
    out = GatedAct{PNV_ACT_SITU, beta, linear_beta, nullptr};
  } else {
    return fail(PNV_ERR_INVALID_ARGUMENT, "activation must be 'silu' or 'situ', got kind %d", act_kind);
  }
  return PNV_OK;
}

}  // namespace pnv

using namespace pnv;

extern "C" int pnv_quant_act(const void* x, const float* gscale, int gscale_per_expert,
                             const int32_t* counts, int experts, int max_n, int k, uint8_t* b_act,
                             uint8_t* sfb, int sm_count, pnv_stream_t stream) {
  if (int rc = check_common(x, gscale, counts, experts, max_n, k, b_act, sfb, "K")) return rc;
  long long lines = sf_numel(max_n, k, experts) / 16;
  GatedAct act{PNV_ACT_SILU, 1.f, -1.f, nullptr};
  PNV_CUDA(launch_pdl(quant_lines_kernel<kPlain>, dim3(grid_for(lines, sm_count)), dim3(kThreads), 0,
                      (cudaStream_t)stream, pdl_enabled(), (const __nv_bfloat16*)x, gscale,
                      gscale_per_expert, counts, experts, max_n, k, 0, act, b_act, sfb));
  return PNV_OK;
}

extern "C" int pnv_silu_mul_quant_act(const void* x2, const float* gscale, int gscale_per_expert,
                                      const int32_t* counts, int experts, int max_n, int n,
                                      int interleaved, int act_kind, float beta, float linear_beta,
                                      uint8_t* b_act, uint8_t* sfb, int sm_count,
                                      pnv_stream_t stream) {
  GatedAct act;
  if (int rc = make_gated_act(act_kind, beta, linear_beta, (cudaStream_t)stream, act)) return rc;
  if (int rc = check_common(x2, gscale, counts, experts, max_n, n, b_act, sfb, "intermediate width N"))
    return rc;
  long long lines = sf_numel(max_n, n, experts) / 16;
  PNV_CUDA(launch_pdl(quant_lines_kernel<kGated>, dim3(grid_for(lines, sm_count)), dim3(kThreads), 0,
                      (cudaStream_t)stream, pdl_enabled(), (const __nv_bfloat16*)x2, gscale,
                      gscale_per_expert, counts, experts, max_n, n, interleaved ? 1 : 0, act,
                      b_act, sfb));
  return PNV_OK;
}

extern "C" int pnv_scatter_quant_act(const void* a1, const int64_t* flat_tok,
                                     const int64_t* dest_global, const float* topk_weights,
                                     const float* gscale, int gscale_per_expert, int64_t n_routes,
                                     int k, int experts, int cap, uint8_t* b_act, uint8_t* sfb,
                                     int sm_count, pnv_stream_t stream) {
  PNV_REQUIRE(cap > 0, "cap must be positive");
  PNV_REQUIRE(n_routes >= 0, "n_routes must be non-negative");
  PNV_REQUIRE(n_routes == 0 || (flat_tok && dest_global), "null routing plan");
  int dummy = 0;
  if (int rc = check_common(a1 ? a1 : (const void*)&dummy, gscale, &dummy, experts, cap, k, b_act, sfb, "K"))
    return rc;
  PNV_REQUIRE(n_routes == 0 || a1, "null pointer argument");
  cudaStream_t s = (cudaStream_t)stream;
  PNV_CUDA(cudaMemsetAsync(sfb, kBenignSf, (size_t)sf_numel(cap, k, experts), s));
  if (n_routes == 0) return PNV_OK;
  PNV_REQUIRE(n_routes < (1LL << 31) && (long long)experts * cap < (1LL << 31), "T * topk and E * cap must fit int32");
  PNV_CUDA(launch_pdl(scatter_quant_kernel, dim3(grid_for(n_routes, sm_count)), dim3(kThreads), 0, s,
                      false, (const __nv_bfloat16*)a1, (const long long*)flat_tok,
                      (const long long*)dest_global, topk_weights, gscale, gscale_per_expert,
                      (unsigned)n_routes, k, experts, cap, b_act, sfb));
  return PNV_OK;
}

extern "C" int pnv_gated_act(const void* x2, int64_t rows, int n, int interleaved, int act_kind,
                             float beta, float linear_beta, void* y, pnv_stream_t stream) {
  GatedAct act;
  if (int rc = make_gated_act(act_kind, beta, linear_beta, (cudaStream_t)stream, act)) return rc;
  PNV_REQUIRE(x2 && y, "null pointer argument");
  PNV_REQUIRE(n > 0 && n % kSfBlock == 0, "intermediate width N must be a multiple of %d, got %d", kSfBlock, n);
  if (rows <= 0) return PNV_OK;
  long long total = rows * (n / 8);
  long long blocks = (total + kThreads - 1) / kThreads;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  gated_act_kernel<<<(unsigned)blocks, kThreads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x2, (long long)rows, n, interleaved ? 1 : 0, act, (__nv_bfloat16*)y);
  PNV_CUDA(cudaGetLastError());
  return PNV_OK;
}

extern "C" int pnv_scatter_quant_act_planned(const void* a1, const int32_t* src_tok, const int32_t* src_route,
                                             const float* topk_weights, const float* gscale, int gscale_per_expert,
                                             const int32_t* counts, int k, int experts, int cap, uint8_t* b_act,
                                             uint8_t* sfb, int sm_count, pnv_stream_t stream) {
  PNV_REQUIRE(cap > 0, "cap must be positive");
  PNV_REQUIRE(src_tok && src_route, "null pointer argument");
  if (int rc = check_common(a1, gscale, counts, experts, cap, k, b_act, sfb, "K")) return rc;
  PNV_REQUIRE((long long)experts * cap < (1LL << 31), "E * cap must fit int32");
  cudaStream_t s = (cudaStream_t)stream;
  // benign fill first, then one warp per live row writes its scales over it
  PNV_CUDA(cudaMemsetAsync(sfb, kBenignSf, (size_t)sf_numel(cap, k, experts), s));
  PNV_CUDA(launch_pdl(scatter_planned_rows_kernel, dim3(grid_for((long long)experts * cap, sm_count)), dim3(kThreads), 0, s,
                      false, (const __nv_bfloat16*)a1, (const int*)src_tok, (const int*)src_route, topk_weights, gscale,
                      gscale_per_expert, (const int*)counts, k, experts, cap, b_act, sfb));
  return PNV_OK;
}

extern "C" int pnv_quant_rows(const void* x, const float* gscale, int64_t tokens, int k, uint8_t* q, uint8_t* q_sf,
                              int sm_count, pnv_stream_t stream) {
  PNV_REQUIRE(k > 0 && k % kSfBlock == 0, "K must be a multiple of %d, got %d", kSfBlock, k);
  PNV_REQUIRE(tokens >= 0, "bad token count");
  if (tokens == 0) return PNV_OK;
  PNV_REQUIRE(x && gscale && q && q_sf, "null pointer argument");
  PNV_REQUIRE(tokens < (1LL << 31), "too many tokens");
  PNV_CUDA(launch_pdl(quant_rows_kernel, dim3(grid_for(tokens, sm_count)), dim3(kThreads), 0, (cudaStream_t)stream,
                      pdl_enabled(), (const __nv_bfloat16*)x, gscale, (unsigned)tokens, k, q, q_sf));
  return PNV_OK;
}

namespace {
int scatter_fp4_rows(const uint8_t* q, long long q_pitch, const uint8_t* q_sf, long long sf_pitch, const int32_t* src_tok,
                     const int32_t* counts, int k, int experts, int cap, uint8_t* b_act, uint8_t* sfb, int sm_count,
                     cudaStream_t s) {
  float dummy = 0.f;
  if (int rc = check_common(q, &dummy, counts, experts, cap, k, b_act, sfb, "K")) return rc;
  PNV_REQUIRE((long long)experts * cap < (1LL << 31), "E * cap must fit int32");
  PNV_REQUIRE((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(b_act) | (uintptr_t)q_pitch) % 16 == 0,
              "code rows must be 16-byte aligned");
  // benign fill first, then one warp per live row writes its scales over it
  PNV_CUDA(cudaMemsetAsync(sfb, kBenignSf, (size_t)sf_numel(cap, k, experts), s));
  PNV_CUDA(launch_pdl(scatter_fp4_rows_kernel, dim3(grid_for((long long)experts * cap, sm_count)), dim3(kThreads), 0, s,
                      false, q, q_pitch, q_sf, sf_pitch, (const int*)src_tok, (const int*)counts, k, experts, cap, b_act,
                      sfb));
  return PNV_OK;
}
}  // namespace

extern "C" int pnv_scatter_fp4_planned(const uint8_t* q, const uint8_t* q_sf, const int32_t* src_tok,
                                       const int32_t* counts, int k, int experts, int cap, uint8_t* b_act,
                                       uint8_t* sfb, int sm_count, pnv_stream_t stream) {
  PNV_REQUIRE(cap > 0, "cap must be positive");
  PNV_REQUIRE(q && q_sf && src_tok, "null pointer argument");
  PNV_REQUIRE(k > 0 && k % kSfBlock == 0, "K must be a multiple of %d, got %d", kSfBlock, k);
  return scatter_fp4_rows(q, k / 2, q_sf, k / kSfBlock, src_tok, counts, k, experts, cap, b_act, sfb, sm_count,
                          (cudaStream_t)stream);
}

extern "C" int pnv_set_silu_table(int enabled) {
  g_silu_table_on = enabled != 0;
  return PNV_OK;
}


extern "C" int64_t pnv_wire_row_bytes(int k) {
  if (k <= 0 || k % kSfBlock != 0) return 0;
  return wire_row_bytes(k);
}

namespace {
int pack_wire_rows_common(const uint8_t* q, const uint8_t* q_sf, const void* topk_ids, int ids_are_int64,
                          const int32_t* slot_tok, const int32_t* slot_route, const int32_t* slab_counts, int ranks,
                          int slab, int experts_per_rank, int k, uint8_t* wire, const RowParts& parts,
                          pnv_stream_t stream) {
  PNV_REQUIRE(k > 0 && k % kSfBlock == 0, "K must be a multiple of %d, got %d", kSfBlock, k);
  PNV_REQUIRE(ranks >= 1 && slab >= 1 && experts_per_rank >= 1, "ranks, slab and experts_per_rank must be positive");
  PNV_REQUIRE((long long)ranks * slab < (1LL << 31), "ranks * slab must fit int32");
  PNV_REQUIRE(q && q_sf && topk_ids && slot_tok && slot_route && slab_counts, "null pointer argument");
  PNV_REQUIRE((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(wire)) % 16 == 0 &&
                  ((k / kSfBlock) % 16 != 0 || reinterpret_cast<uintptr_t>(q_sf) % 16 == 0),
              "pack_wire_rows buffers must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid((unsigned)(ranks * slab)), block(128);
  if (ids_are_int64)
    PNV_CUDA(launch_pdl(pack_wire_rows_kernel<long long>, grid, block, 0, s, pdl_enabled(), q, q_sf,
                        (const long long*)topk_ids, (const int*)slot_tok, (const int*)slot_route,
                        (const int*)slab_counts, slab, experts_per_rank, k, wire, parts));
  else
    PNV_CUDA(launch_pdl(pack_wire_rows_kernel<int>, grid, block, 0, s, pdl_enabled(), q, q_sf, (const int*)topk_ids,
                        (const int*)slot_tok, (const int*)slot_route, (const int*)slab_counts, slab,
                        experts_per_rank, k, wire, parts));
  return PNV_OK;
}
}  // namespace

extern "C" int pnv_pack_wire_rows(const uint8_t* q, const uint8_t* q_sf, const void* topk_ids, int ids_are_int64,
                                  const int32_t* slot_tok, const int32_t* slot_route, const int32_t* slab_counts,
                                  int ranks, int slab, int experts_per_rank, int k, uint8_t* wire,
                                  pnv_stream_t stream) {
  PNV_REQUIRE(wire, "null pointer argument");
  RowParts none{};
  return pack_wire_rows_common(q, q_sf, topk_ids, ids_are_int64, slot_tok, slot_route, slab_counts, ranks, slab,
                               experts_per_rank, k, wire, none, stream);
}

extern "C" int pnv_pack_wire_rows_parts(const uint8_t* q, const uint8_t* q_sf, const void* topk_ids, int ids_are_int64,
                                        const int32_t* slot_tok, const int32_t* slot_route,
                                        const int32_t* slab_counts, int ranks, int slab, int experts_per_rank, int k,
                                        void* const* wire_parts, pnv_stream_t stream) {
  RowParts parts;
  if (int rc = make_row_parts(wire_parts, ranks, slab, parts)) return rc;
  return pack_wire_rows_common(q, q_sf, topk_ids, ids_are_int64, slot_tok, slot_route, slab_counts, ranks, slab,
                               experts_per_rank, k, nullptr, parts, stream);
}

extern "C" int pnv_scatter_fp4_wire(const uint8_t* wire, const int32_t* src_tok, const int32_t* counts, int k,
                                    int experts, int cap, uint8_t* b_act, uint8_t* sfb, int sm_count,
                                    pnv_stream_t stream) {
  PNV_REQUIRE(cap > 0, "cap must be positive");
  PNV_REQUIRE(wire && src_tok, "null pointer argument");
  PNV_REQUIRE(k > 0 && k % kSfBlock == 0, "K must be a multiple of %d, got %d", kSfBlock, k);
  const long long pitch = wire_row_bytes(k);
  return scatter_fp4_rows(wire, pitch, wire + k / 2, pitch, src_tok, counts, k, experts, cap, b_act, sfb, sm_count,
                          (cudaStream_t)stream);
}
