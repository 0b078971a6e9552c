// Load-time weight compressor: dense packed e2m1 [E, M, K/2] + natural-order UE4M3 [E, M, K/32]
// -> the three operands the sparse block-scaled MMA reads:
//   a_comp  [E, M, round_up(K,64)/4]   the two kept bytes (e2m1 pairs) of every 4-byte chunk
//   e_meta  [E, round_up(M,128), round_up(K,256)/16]  one nibble per chunk = the two 2-bit
//           in-chunk indices of the kept bytes, in 128-row x 16-byte atoms (see common.cuh)
//   sfa     swizzled scale atoms, slop bytes zero
//
// A quad of lanes owns one (row, 256-K) metadata line: each lane reads 32 bytes (8 chunks) with
// two 128-bit loads, emits 16 bytes of a_comp with one 128-bit store and 4 bytes of metadata, so
// the quad writes the row's 16-byte metadata line contiguously.
#include "common.cuh"

namespace pnv {
namespace {

constexpr int kThreads = 256;

// One 4-byte chunk (8 e2m1 values) -> (two kept bytes, 4-bit index nibble).
// A byte is "zero" when both magnitudes are zero (sign bits ignored).  Chunks with one non-zero
// byte are padded with a zero byte so that the two indices stay strictly ordered: a lone byte at
// index 3 becomes (0 @0, byte @3), a lone byte at i < 3 becomes (byte @i, 0 @3).
__device__ __forceinline__ void compress_chunk(uint32_t chunk, uint32_t& kept2, uint32_t& nibble) {
  uint32_t b[4] = {chunk & 0xFF, (chunk >> 8) & 0xFF, (chunk >> 16) & 0xFF, chunk >> 24};
  int idx[2] = {0, 0};
  uint32_t val[2] = {0, 0};
  int n = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if ((b[i] & 0x77u) != 0 && n < 2) {
      idx[n] = i;
      val[n] = b[i];
      ++n;
    }
  }
  if (n == 1) {
    if (idx[0] == 3) {
      val[1] = val[0]; val[0] = 0; idx[0] = 0; idx[1] = 3;
    } else {
      idx[1] = 3;
    }
  }
  kept2 = val[0] | (val[1] << 8);
  nibble = (uint32_t)(idx[0] | (idx[1] << 2));
}

__global__ void __launch_bounds__(kThreads)
compress_kernel(const uint8_t* __restrict__ w_packed, int E, int M, int K, WeightDims wd,
                uint8_t* __restrict__ a_comp, uint8_t* __restrict__ e_meta) {
  const int k_atoms = wd.k_e / 16;            // 256-K metadata atoms per row
  const int m_atoms = wd.m_e / 128;
  const int row_bytes_in = K / 2;
  const int row_bytes_ac = wd.k_ac / 2;
  const long long quads = (long long)E * wd.m_e * k_atoms;
  const long long total = quads * 4;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const int q = (int)(t & 3);                // which 64-K quarter of the 256-K line
    long long a = t >> 2;
    const int ka = (int)(a % k_atoms);
    a /= k_atoms;
    const int m = (int)(a % wd.m_e);
    const int e = (int)(a / wd.m_e);
    const int kbyte0 = ka * 128 + q * 32;      // first input byte of this lane
    uint32_t in[8];
    uint32_t out[4] = {0, 0, 0, 0};
    uint32_t meta = 0;
    if (m < M) {
      const uint8_t* src = w_packed + ((long long)e * M + m) * row_bytes_in + kbyte0;
      if (kbyte0 + 32 <= row_bytes_in && (row_bytes_in % 16) == 0) {
        uint4 v0 = __ldg(reinterpret_cast<const uint4*>(src));
        uint4 v1 = __ldg(reinterpret_cast<const uint4*>(src) + 1);
        in[0] = v0.x; in[1] = v0.y; in[2] = v0.z; in[3] = v0.w;
        in[4] = v1.x; in[5] = v1.y; in[6] = v1.z; in[7] = v1.w;
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c)   // K % 8 == 0, so whole 4-byte chunks exist or not
          in[c] = (kbyte0 + c * 4 + 4 <= row_bytes_in) ? __ldg(reinterpret_cast<const uint32_t*>(src) + c) : 0u;
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t kept, nib;
        compress_chunk(in[c], kept, nib);
        out[c >> 1] |= kept << ((c & 1) * 16);
        meta |= nib << (4 * c);
      }
    }
    // metadata line: atom (e, ka, m / 128), row m % 128, 4 bytes per lane
    const long long atom = ((long long)e * k_atoms + ka) * m_atoms + (m >> 7);
    *reinterpret_cast<uint32_t*>(e_meta + atom * 2048 + (m & 127) * 16 + q * 4) = meta;
    const int acbyte0 = ka * 64 + q * 16;
    if (m < M && acbyte0 < row_bytes_ac) {
      *reinterpret_cast<uint4*>(a_comp + ((long long)e * wd.m_ac + m) * row_bytes_ac + acbyte0) =
          make_uint4(out[0], out[1], out[2], out[3]);
    }
  }
}

// One thread per 16-byte line of the swizzled scale buffer (4 rows x 4 K-blocks).
__global__ void __launch_bounds__(kThreads)
swizzle_sfa_kernel(const uint8_t* __restrict__ sf_nat, int E, int M, int KB, int n_rt, int n_kt,
                   uint8_t* __restrict__ sfa) {
  const long long lines = (long long)E * n_rt * n_kt * 32;
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < lines;
       c += (long long)gridDim.x * blockDim.x) {
    const int rr = (int)(c & 31);
    long long a = c >> 5;
    const int kt = (int)(a % n_kt);
    a /= n_kt;
    const int rt = (int)(a % n_rt);
    const int e = (int)(a / n_rt);
    uint32_t w[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int r = rt * 128 + rr + 32 * g;
      uint32_t word = 0;
      if (r < M) {
        const uint8_t* src = sf_nat + ((long long)e * M + r) * KB + kt * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (kt * 4 + i < KB) word |= (uint32_t)__ldg(src + i) << (8 * i);
      }
      w[g] = word;
    }
    *reinterpret_cast<uint4*>(sfa + c * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace
}  // namespace pnv

using namespace pnv;

extern "C" int pnv_compress(const uint8_t* w_packed, const uint8_t* w_blockscale, int experts,
                            int features, int k, uint8_t* a_comp, uint8_t* e_meta, uint8_t* sfa,
                            pnv_stream_t stream) {
  PNV_REQUIRE(w_packed && w_blockscale && a_comp && e_meta && sfa, "null pointer argument");
  PNV_REQUIRE(experts >= 1 && features >= 1, "experts and features must be positive");
  PNV_REQUIRE(k > 0 && k % 8 == 0,
              "compress: K must be a multiple of 8 (whole 4-pair chunks), got %d", k);
  cudaStream_t s = (cudaStream_t)stream;
  WeightDims wd = weight_dims(features, k);
  long long threads = (long long)experts * wd.m_e * (wd.k_e / 16) * 4;
  long long blocks = (threads + kThreads - 1) / kThreads;
  if (blocks > 148LL * 64) blocks = 148LL * 64;
  compress_kernel<<<(unsigned)blocks, kThreads, 0, s>>>(w_packed, experts, features, k, wd, a_comp, e_meta);
  PNV_CUDA(cudaGetLastError());
  const int KB = ceil_div_i(k, kSfBlock);
  const int n_rt = sf_row_atoms(features), n_kt = sf_k_atoms(k);
  long long lines = (long long)experts * n_rt * n_kt * 32;
  blocks = (lines + kThreads - 1) / kThreads;
  if (blocks > 148LL * 64) blocks = 148LL * 64;
  swizzle_sfa_kernel<<<(unsigned)blocks, kThreads, 0, s>>>(w_blockscale, experts, features, KB, n_rt, n_kt, sfa);
  PNV_CUDA(cudaGetLastError());
  return PNV_OK;
}
