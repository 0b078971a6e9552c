// Routing plan and combine: the two steps either side of the expert FFN.
//
// dispatch_plan.  Routing i = t * topk + j goes to local expert e = topk_ids[i] - first_expert (when
// that is in [0, E)); its rank r is the number of earlier routings (smaller i) to the same expert; it
// is kept when r < cap and lands in row e * cap + r.  That is a stable sort of the routings by
// expert, done here in segments of 1024 routings:
//   sort     one block per segment sorts the keys (expert << 10 | position in segment) with a bitonic
//            network (strides below 32 by shuffles, the rest through shared memory).  The position in
//            the low bits makes every key unique, so the unstable network yields the stable order.
//            In the sorted segment the routings of one expert are one run; a run's start found with
//            a max-scan gives every routing its rank inside the segment, and the run's length is the
//            segment's total for that expert.
//   offsets  (plans of more than one segment) exclusive prefix of the totals over segments, one warp
//            per expert, and counts[e] = min(total, cap)
//   place    (plans of more than one segment) rank = rank in segment + offset of (segment, expert)
//            -> route_dest, src_tok, src_route
// A plan that fits one segment is finished by the sort kernel alone.  No global atomics and no
// host reads, so the plan is deterministic and can be captured in a CUDA graph.
//
// moe_finalize.  out[t] = sum over kept routings, in top-k order, of the expert output rows,
// optionally weighted with torch's rounding chain.  One block per token: destination rows and
// (pre-rounded) weights of the token go to shared memory once, then every thread issues the loads
// of all top-k rows of its 8 columns together before it starts adding.
#include <mutex>

#include "common.cuh"

namespace pnv {
namespace {

constexpr int kSeg = 1024;              // routings per segment = threads of the sort block
constexpr int kSegBits = 10;
constexpr int kNotLocal = 0x1FFF;       // expert code of routings to other ranks and of padding: sorts last

__device__ __forceinline__ unsigned cmp_swap(unsigned mine, unsigned other, bool keep_small) {
  return (mine < other) == keep_small ? mine : other;
}

// totals: [segments][E] (nullptr for single-segment plans, which write the final outputs themselves)
template <class IdT>
__global__ void __launch_bounds__(kSeg)
plan_sort_kernel(const IdT* __restrict__ ids, long long id_stride, int n, int topk, int first, int E, int cap,
                 int* __restrict__ totals,
                 int* __restrict__ counts, int* __restrict__ route_dest, int* __restrict__ src_tok,
                 int* __restrict__ src_route) {
  __shared__ unsigned s_key[kSeg];
  __shared__ int s_warp_max[kSeg / 32];
  extern __shared__ int s_total[];      // [E] totals of this segment
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seg0 = blockIdx.x * kSeg;
  for (int x = tid; x < E; x += kSeg) s_total[x] = 0;
  unsigned code = kNotLocal;
  if (seg0 + tid < n) {
    const long long e = (long long)ids[(seg0 + tid) * id_stride] - first;
    if (e >= 0 && e < E) code = (unsigned)e;
  }
  unsigned key = (code << kSegBits) | (unsigned)tid;
  // bitonic sort, ascending, one key per thread
#pragma unroll 1
  for (int k = 2; k <= kSeg; k <<= 1) {
    const bool up = (tid & k) == 0;
#pragma unroll 1
    for (int j = k >> 1; j > 0; j >>= 1) {
      unsigned other;
      if (j >= 32) {
        __syncthreads();
        s_key[tid] = key;
        __syncthreads();
        other = s_key[tid ^ j];
      } else {
        other = __shfl_xor_sync(0xffffffffu, key, j);
      }
      key = cmp_swap(key, other, ((tid & j) == 0) == up);
    }
  }
  // runs of equal expert in the sorted order
  __syncthreads();
  s_key[tid] = key;
  __syncthreads();
  const unsigned my_code = key >> kSegBits;
  const bool head = tid == 0 || (s_key[tid - 1] >> kSegBits) != my_code;
  const bool tail = tid == kSeg - 1 || (s_key[tid + 1] >> kSegBits) != my_code;
  int start = head ? tid : 0;           // inclusive max-scan of the run starts
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, start, o);
    if (lane >= o) start = max(start, v);
  }
  if (lane == 31) s_warp_max[warp] = start;
  __syncthreads();
  if (warp == 0) {
    int m = s_warp_max[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, m, o);
      if (lane >= o) m = max(m, v);
    }
    s_warp_max[lane] = m;
  }
  __syncthreads();
  if (warp > 0) start = max(start, s_warp_max[warp - 1]);
  const int rank = tid - start;         // rank of this routing among its expert's routings of the segment
  const bool local = my_code != (unsigned)kNotLocal;
  if (local && tail) s_total[my_code] = rank + 1;
  const int i = seg0 + (int)(key & (kSeg - 1));      // the routing this sorted slot holds
  if (totals != nullptr) {
    // several segments: leave the rank in the segment for the place pass
    if (i < n) route_dest[i] = local ? rank : -1;
    __syncthreads();
    for (int x = tid; x < E; x += kSeg) totals[(long long)blockIdx.x * E + x] = s_total[x];
  } else {
    if (i < n) {
      int dest = -1;
      if (local && rank < cap) {
        dest = (int)my_code * cap + rank;
        src_tok[dest] = i / topk;
        src_route[dest] = i;
      }
      route_dest[i] = dest;
    }
    __syncthreads();
    for (int x = tid; x < E; x += kSeg) counts[x] = min(s_total[x], cap);
  }
}

// totals[segment][e] -> exclusive prefix over segments, in place; counts[e] = min(total, cap).
// One warp per expert, 32 segments per step.
__global__ void __launch_bounds__(256)
plan_offsets_kernel(int* __restrict__ totals, int segments, int E, int cap, int* __restrict__ counts) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int e = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (e >= E) return;
  int carry = 0;
  for (int s0 = 0; s0 < segments; s0 += 32) {
    const int s = s0 + lane;
    const int v = s < segments ? totals[(long long)s * E + e] : 0;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += u;
    }
    if (s < segments) totals[(long long)s * E + e] = carry + incl - v;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) counts[e] = min(carry, cap);
}

template <class IdT>
__global__ void __launch_bounds__(256)
plan_place_kernel(const IdT* __restrict__ ids, long long id_stride, int n, int topk, int first, int E, int cap,
                  const int* __restrict__ offsets, int* __restrict__ route_dest, int* __restrict__ src_tok,
                  int* __restrict__ src_route) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int in_seg = route_dest[i];
  int dest = -1;
  if (in_seg >= 0) {
    const int e = (int)((long long)ids[i * id_stride] - first);
    const int r = in_seg + offsets[(long long)(i >> kSegBits) * E + e];
    if (r < cap) {
      dest = e * cap + r;
      src_tok[dest] = i / topk;
      src_route[dest] = i;
    }
  }
  route_dest[i] = dest;
}

template <class IdT>
int run_plan(const IdT* ids, long long id_stride, int n, int topk, int first, int E, int cap, int* counts, int* route_dest,
             int* src_tok, int* src_route, int* scratch, cudaStream_t s) {
  const int segments = (n + kSeg - 1) / kSeg;
  if (segments == 0) {
    PNV_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * (size_t)E, s));
    return PNV_OK;
  }
  const size_t smem = sizeof(int) * (size_t)E;     // static shared memory takes 4.1 KiB more: always below 48 KiB
  const bool pdl = pdl_enabled();
  if (segments == 1) {
    PNV_CUDA(launch_pdl(plan_sort_kernel<IdT>, dim3(1), dim3(kSeg), smem, s, pdl, ids, id_stride, n, topk, first, E, cap,
                        (int*)nullptr, counts, route_dest, src_tok, src_route));
    return PNV_OK;
  }
  PNV_REQUIRE(scratch != nullptr, "dispatch_plan: %d segments need a scratch buffer of segments * E ints", segments);
  PNV_CUDA(launch_pdl(plan_sort_kernel<IdT>, dim3(segments), dim3(kSeg), smem, s, pdl, ids, id_stride, n, topk, first, E, cap,
                      scratch, counts, route_dest, src_tok, src_route));
  PNV_CUDA(launch_pdl(plan_offsets_kernel, dim3((E + 7) / 8), dim3(256), 0, s, pdl, scratch, segments, E, cap, counts));
  PNV_CUDA(launch_pdl(plan_place_kernel<IdT>, dim3((n + 255) / 256), dim3(256), 0, s, pdl, ids, id_stride, n, topk, first, E, cap,
                      (const int*)scratch, route_dest, src_tok, src_route));
  return PNV_OK;
}

// Built-in scratch for pnv_dispatch_plan_noalloc: per-segment expert totals, segments * E ints, at most
// kBuiltinScratchInts (256 KiB).  It lives in every GPU that loads the library until the process
// exits.  In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
constexpr int kBuiltinScratchInts = 65536;
static __device__ __align__(256) int g_plan_scratch[kBuiltinScratchInts];

// Device address of g_plan_scratch on the current device, looked up once per device.
int builtin_scratch(int** out) {
  static std::mutex mu;
  static int* ptrs[64] = {};
  int dev = 0;
  PNV_CUDA(cudaGetDevice(&dev));
  PNV_REQUIRE(dev >= 0 && dev < 64, "unexpected CUDA device index %d", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    int* p = nullptr;
    PNV_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_plan_scratch));
    PNV_REQUIRE(p != nullptr, "cudaGetSymbolAddress returned a null address for the built-in scratch");
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return PNV_OK;
}

constexpr int kFinThreads = 256;
constexpr int kFinMaxTopk = 32;         // routings of a token staged in shared memory at a time

// TOPK > 0: the token's top-k row loads of one 16-byte column group are all issued before the first add.
template <int TOPK>
__global__ void __launch_bounds__(kFinThreads)
finalize_kernel(const uint4* __restrict__ fused, const int* __restrict__ route_dest, const float* __restrict__ topk_w,
                uint4* __restrict__ out, int topk, int vecs) {
  __shared__ int s_dest[kFinMaxTopk];
  __shared__ float s_w[kFinMaxTopk];
  pdl_wait();
  pdl_launch_dependents();
  const long long t = blockIdx.x;
  const int nk = TOPK > 0 ? TOPK : topk;
  // dropped routings (dest < 0) are never read; the weight is rounded to bf16 once, as torch would
  if constexpr (TOPK > 0) {
    if (threadIdx.x < TOPK) {
      s_dest[threadIdx.x] = route_dest[t * TOPK + threadIdx.x];
      s_w[threadIdx.x] = topk_w ? __bfloat162float(__float2bfloat16_rn(topk_w[t * TOPK + threadIdx.x])) : 1.f;
    }
    __syncthreads();
  }
  const bool weighted = topk_w != nullptr;
  for (int v = threadIdx.x; v < vecs; v += kFinThreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if constexpr (TOPK > 0) {
      uint4 r[TOPK];
#pragma unroll
      for (int k = 0; k < TOPK; ++k) {
        const int d = s_dest[k];
        r[k] = d >= 0 ? __ldg(fused + (long long)d * vecs + v) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int k = 0; k < TOPK; ++k) {
        if (s_dest[k] < 0) continue;
        float x[8];
        unpack8(r[k], x);
        if (weighted) {
          const float w = s_w[k];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], __bfloat162float(__float2bfloat16_rn(__fmul_rn(x[j], w))));
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], x[j]);
        }
      }
    } else {
      for (int k = 0; k < nk; ++k) {
        const int d = route_dest[t * nk + k];
        if (d < 0) continue;
        float x[8];
        unpack8(__ldg(fused + (long long)d * vecs + v), x);
        if (weighted) {
          const float w = __bfloat162float(__float2bfloat16_rn(topk_w[t * nk + k]));
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], __bfloat162float(__float2bfloat16_rn(__fmul_rn(x[j], w))));
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], x[j]);
        }
      }
    }
    __nv_bfloat16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(acc[j]);
    out[t * vecs + v] = *reinterpret_cast<const uint4*>(o);
  }
}

// gather_rows: dst[i, :] = idx[i] >= 0 ? src[idx[i], :] : 0, rows of `vecs` 16-byte words; one block
// per destination row.  The copy step either side of an expert-parallel exchange: token rows into
// send order, expert output rows into return order (dropped routings come back as zero rows).
constexpr int kGatherThreads = 128;

__global__ void __launch_bounds__(kGatherThreads)
gather_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ idx, uint4* __restrict__ dst, int vecs) {
  pdl_wait();
  pdl_launch_dependents();
  const long long i = blockIdx.x;
  const int r = idx[i];
  uint4* out = dst + i * vecs;
  if (r < 0) {
    for (int v = threadIdx.x; v < vecs; v += kGatherThreads) out[v] = make_uint4(0u, 0u, 0u, 0u);
  } else {
    const uint4* in = src + (long long)r * vecs;
    for (int v = threadIdx.x; v < vecs; v += kGatherThreads) out[v] = __ldg(in + v);
  }
}

// zero_rows: rows whose flag is negative become zero, the others are left alone; one warp per row.  With
// group_mm_rows (expert output rows written straight into return order) this stands in for gather_rows:
// the slots no expert row lands on (dropped and dead ones) still return zeros.
__global__ void __launch_bounds__(256)
zero_rows_kernel(const int* __restrict__ flags, long long rows, uint4* __restrict__ dst, int vecs, const RowParts parts) {
  pdl_wait();
  pdl_launch_dependents();
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= rows || flags[r] >= 0) return;
  uint4* out = parts.n ? reinterpret_cast<uint4*>(part_row(parts, r, (long long)vecs * 16)) : dst + r * vecs;
  for (int v = threadIdx.x & 31; v < vecs; v += 32) out[v] = make_uint4(0u, 0u, 0u, 0u);
}

}  // namespace
}  // namespace pnv

using namespace pnv;

extern "C" int64_t pnv_dispatch_plan_scratch_ints(int64_t n_routes, int num_local_experts) {
  if (n_routes < 0 || num_local_experts < 1) return 0;
  const int64_t segments = (n_routes + kSeg - 1) / kSeg;
  return segments > 1 ? segments * num_local_experts : 0;
}

namespace {
// The argument checks both plan entry points share; everything is validated before any size is derived.
int check_plan_args(const void* topk_ids, int64_t tokens, int topk, int num_local_experts, int cap,
                    const int32_t* counts, const int32_t* route_dest, const int32_t* src_tok, const int32_t* src_route) {
  PNV_REQUIRE(num_local_experts >= 1 && num_local_experts <= 4096, "num_local_experts must be in [1, 4096], got %d",
              num_local_experts);
  PNV_REQUIRE(cap >= 1, "cap must be positive");
  PNV_REQUIRE((long long)num_local_experts * cap < (1LL << 31), "E * cap must fit int32");
  PNV_REQUIRE(tokens >= 0 && topk >= 1 && tokens < (1LL << 31) && tokens * topk < (1LL << 31),
              "T * topk must fit int32");
  PNV_REQUIRE(counts && (tokens == 0 || (topk_ids && route_dest && src_tok && src_route)), "null pointer argument");
  return PNV_OK;
}
}  // namespace

extern "C" int pnv_dispatch_plan_strided(const void* topk_ids, int ids_are_int64, int64_t id_stride, int64_t tokens,
                                         int topk, int first_expert, int num_local_experts, int cap, int32_t* counts,
                                         int32_t* route_dest, int32_t* src_tok, int32_t* src_route, int32_t* scratch,
                                         pnv_stream_t stream) {
  if (int rc = check_plan_args(topk_ids, tokens, topk, num_local_experts, cap, counts, route_dest, src_tok, src_route))
    return rc;
  PNV_REQUIRE(id_stride >= 1, "id_stride must be positive");
  const int n = (int)(tokens * topk);
  cudaStream_t s = (cudaStream_t)stream;
  if (ids_are_int64)
    return run_plan(static_cast<const long long*>(topk_ids), (long long)id_stride, n, topk, first_expert,
                    num_local_experts, cap, counts, route_dest, src_tok, src_route, scratch, s);
  return run_plan(static_cast<const int*>(topk_ids), (long long)id_stride, n, topk, first_expert, num_local_experts, cap,
                  counts, route_dest, src_tok, src_route, scratch, s);
}

extern "C" int pnv_dispatch_plan(const void* topk_ids, int ids_are_int64, int64_t tokens, int topk, int first_expert,
                                 int num_local_experts, int cap, int32_t* counts, int32_t* route_dest,
                                 int32_t* src_tok, int32_t* src_route, int32_t* scratch, pnv_stream_t stream) {
  return pnv_dispatch_plan_strided(topk_ids, ids_are_int64, 1, tokens, topk, first_expert, num_local_experts, cap, counts,
                                   route_dest, src_tok, src_route, scratch, stream);
}

extern "C" int64_t pnv_dispatch_plan_noalloc_max_scratch_ints(void) { return kBuiltinScratchInts; }

extern "C" int pnv_dispatch_plan_noalloc(const void* topk_ids, int ids_are_int64, int64_t tokens, int topk,
                                         int first_expert, int num_local_experts, int cap, int32_t* counts,
                                         int32_t* route_dest, int32_t* src_tok, int32_t* src_route,
                                         pnv_stream_t stream) {
  if (int rc = check_plan_args(topk_ids, tokens, topk, num_local_experts, cap, counts, route_dest, src_tok, src_route))
    return rc;
  const int64_t need = pnv_dispatch_plan_scratch_ints(tokens * topk, num_local_experts);
  PNV_REQUIRE(need <= kBuiltinScratchInts,
              "dispatch_plan_noalloc: %lld routings over %d local experts need %lld scratch ints, the built-in "
              "scratch holds %d; use pnv_dispatch_plan with a caller-provided buffer",
              (long long)(tokens * topk), num_local_experts, (long long)need, kBuiltinScratchInts);
  // The array belongs to the current device; a stream of another device would make the kernels run where
  // this address means nothing.
  int dev = 0, stream_dev = 0;
  PNV_CUDA(cudaGetDevice(&dev));
  if (stream != nullptr && cudaStreamGetDevice((cudaStream_t)stream, &stream_dev) == cudaSuccess)
    PNV_REQUIRE(stream_dev == dev, "dispatch_plan_noalloc: the stream belongs to device %d, the current device is %d",
                stream_dev, dev);
  int* scratch = nullptr;
  if (int rc = builtin_scratch(&scratch)) return rc;
  // Nothing in the scratch has to start at zero: the sort pass writes every total of every segment
  // this plan uses before the scan reads it, so whatever an earlier call left behind is ignored.
  return pnv_dispatch_plan(topk_ids, ids_are_int64, tokens, topk, first_expert, num_local_experts, cap, counts,
                           route_dest, src_tok, src_route, scratch, stream);
}

extern "C" int pnv_moe_finalize(void* out, const void* fused, const int32_t* route_dest, const float* topk_weights,
                                int64_t tokens, int topk, int k, pnv_stream_t stream) {
  PNV_REQUIRE(k > 0 && k % 8 == 0, "K must be a multiple of 8");
  PNV_REQUIRE(tokens >= 0 && topk >= 1, "bad token count or topk");
  if (tokens == 0) return PNV_OK;
  PNV_REQUIRE(out && fused && route_dest, "null pointer argument");
  PNV_REQUIRE(tokens < (1LL << 31), "too many tokens");
  const int vecs = k / 8;
  cudaStream_t s = (cudaStream_t)stream;
  const bool pdl = pdl_enabled();
  const dim3 grid((unsigned)tokens), block(kFinThreads);
  const uint4* f = (const uint4*)fused;
  uint4* o = (uint4*)out;
  const int* rd = (const int*)route_dest;
  switch (topk) {
    case 1: PNV_CUDA(launch_pdl(finalize_kernel<1>, grid, block, 0, s, pdl, f, rd, topk_weights, o, topk, vecs)); break;
    case 2: PNV_CUDA(launch_pdl(finalize_kernel<2>, grid, block, 0, s, pdl, f, rd, topk_weights, o, topk, vecs)); break;
    case 4: PNV_CUDA(launch_pdl(finalize_kernel<4>, grid, block, 0, s, pdl, f, rd, topk_weights, o, topk, vecs)); break;
    case 6: PNV_CUDA(launch_pdl(finalize_kernel<6>, grid, block, 0, s, pdl, f, rd, topk_weights, o, topk, vecs)); break;
    case 8: PNV_CUDA(launch_pdl(finalize_kernel<8>, grid, block, 0, s, pdl, f, rd, topk_weights, o, topk, vecs)); break;
    default: PNV_CUDA(launch_pdl(finalize_kernel<0>, grid, block, 0, s, pdl, f, rd, topk_weights, o, topk, vecs)); break;
  }
  return PNV_OK;
}

extern "C" int pnv_gather_rows(const void* src, const int32_t* idx, int64_t n_idx, int64_t row_bytes, void* dst,
                               pnv_stream_t stream) {
  PNV_REQUIRE(n_idx >= 0 && n_idx < (1LL << 31), "bad row count");
  PNV_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && row_bytes / 16 < (1LL << 31),
              "row_bytes must be a positive multiple of 16, got %lld", (long long)row_bytes);
  if (n_idx == 0) return PNV_OK;
  PNV_REQUIRE(src && idx && dst, "null pointer argument");
  PNV_REQUIRE((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) % 16 == 0,
              "gather_rows buffers must be 16-byte aligned");
  PNV_CUDA(launch_pdl(gather_rows_kernel, dim3((unsigned)n_idx), dim3(kGatherThreads), 0, (cudaStream_t)stream,
                      pdl_enabled(), (const uint4*)src, (const int*)idx, (uint4*)dst, (int)(row_bytes / 16)));
  return PNV_OK;
}

namespace {
int zero_rows_common(void* dst, const RowParts& parts, const int32_t* flags, int64_t rows, int64_t row_bytes,
                     pnv_stream_t stream) {
  PNV_REQUIRE(rows >= 0 && rows < (1LL << 33), "bad row count");
  PNV_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && row_bytes / 16 < (1LL << 31),
              "row_bytes must be a positive multiple of 16, got %lld", (long long)row_bytes);
  if (rows == 0) return PNV_OK;
  PNV_REQUIRE(flags, "null pointer argument");
  PNV_REQUIRE(reinterpret_cast<uintptr_t>(dst) % 16 == 0, "zero_rows buffer must be 16-byte aligned");
  PNV_CUDA(launch_pdl(zero_rows_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, (cudaStream_t)stream,
                      pdl_enabled(), (const int*)flags, (long long)rows, (uint4*)dst, (int)(row_bytes / 16), parts));
  return PNV_OK;
}
}  // namespace

extern "C" int pnv_zero_rows(void* dst, const int32_t* flags, int64_t rows, int64_t row_bytes, pnv_stream_t stream) {
  PNV_REQUIRE(dst || rows == 0, "null pointer argument");
  RowParts none{};
  return zero_rows_common(dst, none, flags, rows, row_bytes, stream);
}

extern "C" int pnv_zero_rows_parts(void* const* parts, int n_parts, int64_t rows_per_part, const int32_t* flags,
                                   int64_t row_bytes, pnv_stream_t stream) {
  RowParts rp;
  if (int rc = make_row_parts(parts, n_parts, rows_per_part, rp)) return rc;
  return zero_rows_common(nullptr, rp, flags, (int64_t)n_parts * rows_per_part, row_bytes, stream);
}
