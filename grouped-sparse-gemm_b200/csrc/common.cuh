// Shared host/device helpers: error reporting for the C ABI, the closed-form operand layouts and
// the numeric conversions every producer shares.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/paired_nvfp4_b200.h"

namespace pnv {

// ---- error reporting -------------------------------------------------------------------------

char* last_error_buffer();   // thread-local, 512 bytes (abi.cu)

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define PNV_REQUIRE(cond, ...)                                             \
  do {                                                                     \
    if (!(cond)) return ::pnv::fail(PNV_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

#define PNV_CUDA(expr)                                                                       \
  do {                                                                                       \
    cudaError_t err__ = (expr);                                                              \
    if (err__ != cudaSuccess)                                                                \
      return ::pnv::fail(PNV_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__));   \
  } while (0)

// ---- layout arithmetic -------------------------------------------------------------------------
//
// Scale-factor buffers (SFA for weights, SFB for activations): one UE4M3 byte per 32 dense K
// elements, stored in 512-byte atoms of 128 rows x 4 K-blocks; K atoms innermost, then row atoms,
// then experts.  Inside an atom the scale of (row r, K-block kb) sits at byte
// (r % 32) * 16 + (r / 32 % 4) * 4 + kb % 4: 32 lines of 16 bytes, which is exactly the source
// shape of one tcgen05.cp.32x128b.warpx4 copy into tensor memory.
//
// Sparsity metadata: 4 bits per 8 dense K elements, two nibbles per byte, in atoms of
// 128 rows x 16 bytes (256 dense K), row-major inside, atoms ordered M-fastest, then K, then
// expert: the source shape of one tcgen05.cp.128x128b copy.

constexpr int kSfBlock = 32;         // dense K elements per scale
constexpr int kBenignSf = 0x38;      // UE4M3 1.0

__host__ __device__ inline int ceil_div_i(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline int round_up_i(int a, int b) { return ceil_div_i(a, b) * b; }

struct WeightDims {
  int m_ac;        // rows of a_comp
  int k_ac;        // e2m1 elements per a_comp row (bytes = k_ac / 2)
  int m_e;         // rows of e_meta
  int k_e;         // bytes per e_meta row
};

__host__ __device__ inline WeightDims weight_dims(int features, int k) {
  return WeightDims{features, round_up_i(k, 64) / 2, round_up_i(features, 128), round_up_i(k, 256) / 16};
}

__host__ __device__ inline int sf_row_atoms(int rows) { return ceil_div_i(rows, 128); }
__host__ __device__ inline int sf_k_atoms(int k) { return ceil_div_i(ceil_div_i(k, kSfBlock), 4); }
__host__ __device__ inline long long sf_numel(int rows, int k, int groups) {
  return (long long)groups * sf_row_atoms(rows) * sf_k_atoms(k) * 512;
}
// Byte offset of scale (group g, row r, K-block kb).
__host__ __device__ inline long long sf_offset(int g, int r, int kb, int n_rt, int n_kt) {
  long long atom = ((long long)g * n_rt + (r >> 7)) * n_kt + (kb >> 2);
  return atom * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3);
}

// ---- outputs spread over several buffers ---------------------------------------------------------
//
// Row q of a logical [n * rows_per_part, width] output lives at row q % rows_per_part of buffer q / rows_per_part.
// The buffers may be another GPU's memory mapped into this process (peer access): the expert-parallel exchange
// lets the producing kernel store every row straight into the buffer of the rank that wants it.
constexpr int kMaxRowParts = 16;
struct RowParts {
  void* base[kMaxRowParts];
  int n;                 // 0: a single buffer, addressed the ordinary way
  int rows_per_part;
};
inline int make_row_parts(void* const* parts, int n_parts, long long rows_per_part, RowParts& out) {
  PNV_REQUIRE(parts != nullptr, "null pointer argument");
  PNV_REQUIRE(n_parts >= 1 && n_parts <= kMaxRowParts, "between 1 and %d output parts, got %d", kMaxRowParts, n_parts);
  PNV_REQUIRE(rows_per_part >= 1 && rows_per_part < (1LL << 31), "bad rows_per_part");
  for (int i = 0; i < kMaxRowParts; ++i) out.base[i] = i < n_parts ? parts[i] : nullptr;
  for (int i = 0; i < n_parts; ++i)
    PNV_REQUIRE(parts[i] != nullptr && reinterpret_cast<uintptr_t>(parts[i]) % 16 == 0, "output part %d is null or not 16-byte aligned", i);
  out.n = n_parts;
  out.rows_per_part = (int)rows_per_part;
  return PNV_OK;
}
// Address of byte 0 of row q (rows of `pitch` bytes).
__device__ __forceinline__ uint8_t* part_row(const RowParts& parts, long long q, long long pitch) {
  const int w = (int)(q / parts.rows_per_part);
  return static_cast<uint8_t*>(parts.base[w]) + (q - (long long)w * parts.rows_per_part) * pitch;
}

// ---- programmatic dependent launch -----------------------------------------------------------

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

bool pdl_enabled();   // env PAIRED_NVFP4_PDL, read once (abi.cu)

// Launch `kernel` so that it may start before its stream predecessor has drained; the kernel
// calls pdl_wait() before its first read of anything the predecessor wrote.
template <class... KArgs, class... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- numeric conversions ------------------------------------------------------------------------

// Two floats -> two e2m1 nibbles (lo in bits 0-3), round-to-nearest-even, saturating to +-6.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{\n\t.reg .b8 b;\n\tcvt.rn.satfinite.e2m1x2.f32 b, %2, %1;\n\tcvt.u32.u8 %0, b;\n\t}"
      : "=r"(r) : "f"(lo), "f"(hi));
  return r;
}

// Eight floats -> one 32-bit word of e2m1 nibbles, element j in nibble j.
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float (&v)[8]) {
  return cvt_e2m1x2(v[0], v[1]) | (cvt_e2m1x2(v[2], v[3]) << 8) | (cvt_e2m1x2(v[4], v[5]) << 16) |
         (cvt_e2m1x2(v[6], v[7]) << 24);
}

// float -> UE4M3 byte, round-to-nearest-even, saturating to 448.
__device__ __forceinline__ uint32_t cvt_ue4m3(float x) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(x));
  return (uint32_t)(r & 0xFF);
}

__device__ __forceinline__ float ue4m3_to_float(uint32_t b) {
  uint32_t h2;
  asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(h2) : "r"(b & 0xFFu));
  __half lo = __ushort_as_half((unsigned short)(h2 & 0xFFFF));
  return __half2float(lo);
}

// The block-scale step every quantizer shares: from the block's amax and the expert's global
// scale g, the stored UE4M3 byte and the multiplier applied before the e2m1 rounding.
//   bsf = amax > 0 ? amax / 6 : 1;  sf = ue4m3(bsf * g);  inv = float(sf) > 0 ? g / float(sf) : 0
__device__ __forceinline__ void block_scale(float amax, float g, uint32_t& sf_byte, float& inv) {
  float bsf = amax > 0.f ? __fdiv_rn(amax, 6.f) : 1.f;
  sf_byte = cvt_ue4m3(__fmul_rn(bsf, g));
  float sf = ue4m3_to_float(sf_byte);
  inv = sf > 0.f ? __fdiv_rn(g, sf) : 0.f;
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// Eight bf16 (one 128-bit word) -> floats, and eight floats -> one word of e2m1 codes after scaling.
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

__device__ __forceinline__ uint32_t quant8(const float (&f)[8], float inv) {
  float s[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i] = __fmul_rn(f[i], inv);
  return cvt_e2m1x8(s);
}

// The gated activation applied between the two expert GEMMs, with the rounding chain of the
// unfused path: silu  -> bf16(float(bf16(g / (1 + expf(-g)))) * u)
//               situ  -> bf16((0.5 b) tanhf(g / b) (1 + tanhf(g / 2)) * (l > 0 ? l tanhf(u / l) : u))
struct GatedAct {
  int kind;
  float beta;
  float linear_beta;
  const uint16_t* silu_tab;   // optional: bf16 bits of silu(g) for every bf16 g (65536 entries), or nullptr
};

static __device__ __noinline__ float situ_act(float g, float u, float beta, float linear_beta) {
  float inv_beta = __fdiv_rn(1.0f, beta);
  float gate_out = __fmul_rn(__fmul_rn(__fmul_rn(0.5f, beta), tanhf(__fmul_rn(g, inv_beta))),
                             __fadd_rn(1.0f, tanhf(__fmul_rn(g, 0.5f))));
  float up_out = linear_beta > 0.0f ? __fmul_rn(linear_beta, tanhf(__fmul_rn(u, __fdiv_rn(1.0f, linear_beta)))) : u;
  return __bfloat162float(__float2bfloat16_rn(__fmul_rn(gate_out, up_out)));
}

// bf16(g / (1 + expf(-g))) for a gate value that is itself a bf16 number.
__device__ __forceinline__ float silu_direct(float g) {
  float s = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
  return __bfloat162float(__float2bfloat16_rn(s));
}
// The same through the table: the gate has only 65536 possible values, and the table is filled with
// silu_direct on the device, so both give the same bits.  One cached load replaces expf, an IEEE
// division (whose slow-path branch also keeps the compiler from interleaving neighbouring
// elements) and a rounding.
__device__ __forceinline__ float silu_lookup(float g, const uint16_t* tab) {
  return __uint_as_float((uint32_t)__ldg(tab + (__float_as_uint(g) >> 16)) << 16);
}
__device__ __forceinline__ float silu_mul(float g, float u, const uint16_t* tab) {
  return __bfloat162float(__float2bfloat16_rn(__fmul_rn(silu_lookup(g, tab), u)));
}

// General form (any activation kind, with or without the table).  SiLU is the hot case and stays
// inline; SiTU is a call, so a caller's unrolled loop stays small.
__device__ __forceinline__ float gated_act(float g, float u, const GatedAct& a) {
  if (a.kind == PNV_ACT_SITU) return situ_act(g, u, a.beta, a.linear_beta);
  float s_bf = a.silu_tab != nullptr ? silu_lookup(g, a.silu_tab) : silu_direct(g);
  return __bfloat162float(__float2bfloat16_rn(__fmul_rn(s_bf, u)));
}

// (activation kind, beta, linear_beta) -> GatedAct with the reference's argument checks; for SiLU it also
// makes sure the lookup table of the current device is filled before anything later on `stream` runs (quant.cu)
int make_gated_act(int act_kind, float beta, float linear_beta, cudaStream_t stream, GatedAct& out);

}  // namespace pnv
