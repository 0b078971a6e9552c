// Routing plan and combine: the two steps either side of the expert FFN.
//
// dispatch_plan: a stable counting sort of the routings by local expert.  Routing i = t*topk + j
// gets rank r = number of earlier routings to the same local expert; it is kept when r < cap and
// lands in row e*cap + r.  Chunks of 1024 routings, one per thread:
//   tally   (plans with more than one chunk) per-chunk totals per expert
//   offsets (plans with more than one chunk) exclusive scan of the totals over chunks, and counts
//   place   rank inside the chunk (match_any inside a warp + a per-warp tally in shared memory)
//           plus the chunk's offset -> route_dest, src_tok, src_route (and counts when 1 chunk)
// No atomics, so the plan is deterministic; nothing syncs, so it can be captured in a graph.
//
// moe_finalize: out[t] = sum over kept routings, in top-k order, of the expert output rows,
// optionally weighted with torch's rounding chain; one thread per 8 output columns.
#include <mutex>

#include "common.cuh"

namespace pnv {
namespace {

constexpr int kChunk = 1024;            // routings per block, one per thread
constexpr int kWarps = kChunk / 32;

template <class IdT>
__device__ __forceinline__ int local_expert_of(const IdT* ids, long long i, long long n, int first, int E) {
  if (i >= n) return E;                 // padding lanes fall in the "not local" bucket
  long long e = (long long)ids[i] - first;
  return (e >= 0 && e < E) ? (int)e : E;
}

// Fills tally[warp][e] (uint16) with the number of lanes of each warp routing to e, and returns this
// thread's expert and its rank among the earlier lanes of its own warp with the same expert.
template <class IdT>
__device__ __forceinline__ void warp_tally(const IdT* ids, long long n, int first, int E, uint16_t* tally,
                                           int& e_out, int& lane_rank) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int j = tid; j < kWarps * E; j += kChunk) tally[j] = 0;
  __syncthreads();
  const int e = local_expert_of(ids, (long long)blockIdx.x * kChunk + tid, n, first, E);
  const unsigned same = __match_any_sync(0xffffffffu, e);
  lane_rank = __popc(same & ((1u << lane) - 1u));
  if (e < E && lane_rank == 0) tally[warp * E + e] = (uint16_t)__popc(same);
  __syncthreads();
  e_out = e;
}

template <class IdT>
__global__ void __launch_bounds__(kChunk)
plan_tally_kernel(const IdT* __restrict__ ids, long long n, int first, int E, int* __restrict__ totals) {
  extern __shared__ uint16_t tally[];
  pdl_wait();
  pdl_launch_dependents();
  int e, lane_rank;
  warp_tally(ids, n, first, E, tally, e, lane_rank);
  for (int x = threadIdx.x; x < E; x += kChunk) {
    int sum = 0;
    for (int w = 0; w < kWarps; ++w) sum += tally[w * E + x];
    totals[(long long)blockIdx.x * E + x] = sum;
  }
}

// totals[chunk][e] -> exclusive prefix over chunks (in place); counts[e] = min(total, cap).
__global__ void plan_offsets_kernel(int* __restrict__ totals, int chunks, int E, int cap, int* __restrict__ counts) {
  pdl_wait();
  pdl_launch_dependents();
  for (int x = blockIdx.x * blockDim.x + threadIdx.x; x < E; x += gridDim.x * blockDim.x) {
    int run = 0;
    for (int c = 0; c < chunks; ++c) {
      const int v = totals[(long long)c * E + x];
      totals[(long long)c * E + x] = run;
      run += v;
    }
    counts[x] = min(run, cap);
  }
}

template <class IdT>
__global__ void __launch_bounds__(kChunk)
plan_place_kernel(const IdT* __restrict__ ids, long long n, int topk, int first, int E, int cap,
                  const int* __restrict__ offsets, int* __restrict__ counts, int* __restrict__ route_dest,
                  int* __restrict__ src_tok, int* __restrict__ src_route) {
  extern __shared__ uint16_t tally[];
  pdl_wait();
  pdl_launch_dependents();
  int e, lane_rank;
  warp_tally(ids, n, first, E, tally, e, lane_rank);
  // exclusive prefix over the warps of this chunk, per expert, in place
  for (int x = threadIdx.x; x < E; x += kChunk) {
    int run = 0;
    for (int w = 0; w < kWarps; ++w) {
      const int v = tally[w * E + x];
      tally[w * E + x] = (uint16_t)run;
      run += v;
    }
    if (offsets == nullptr) counts[x] = min(run, cap);   // single chunk: run is the total
  }
  __syncthreads();
  const long long i = (long long)blockIdx.x * kChunk + threadIdx.x;
  if (i >= n) return;
  int dest = -1;
  if (e < E) {
    const int r = lane_rank + tally[(threadIdx.x >> 5) * E + e] +
                  (offsets != nullptr ? offsets[(long long)blockIdx.x * E + e] : 0);
    if (r < cap) {
      dest = e * cap + r;
      src_tok[dest] = (int)(i / topk);
      src_route[dest] = (int)i;
    }
  }
  route_dest[i] = dest;
}

template <class IdT>
int run_plan(const IdT* ids, long long n, int topk, int first, int E, int cap, int* counts, int* route_dest,
             int* src_tok, int* src_route, int* scratch, cudaStream_t s) {
  const int chunks = (int)((n + kChunk - 1) / kChunk);
  if (chunks == 0) {
    PNV_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * (size_t)E, s));
    return PNV_OK;
  }
  const size_t smem = sizeof(uint16_t) * (size_t)kWarps * (size_t)E;
  if (smem > 48 * 1024) {
    PNV_CUDA(cudaFuncSetAttribute(plan_place_kernel<IdT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PNV_CUDA(cudaFuncSetAttribute(plan_tally_kernel<IdT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  const bool pdl = pdl_enabled();
  const int* offsets = nullptr;
  if (chunks > 1) {
    PNV_REQUIRE(scratch != nullptr, "dispatch_plan: %d chunks need a scratch buffer of chunks * E ints", chunks);
    PNV_CUDA(launch_pdl(plan_tally_kernel<IdT>, dim3(chunks), dim3(kChunk), smem, s, pdl, ids, n, first, E, scratch));
    PNV_CUDA(launch_pdl(plan_offsets_kernel, dim3((E + 255) / 256), dim3(256), 0, s, pdl, scratch, chunks, E, cap,
                        counts));
    offsets = scratch;
  }
  PNV_CUDA(launch_pdl(plan_place_kernel<IdT>, dim3(chunks), dim3(kChunk), smem, s, pdl, ids, n, topk, first, E, cap,
                      offsets, counts, route_dest, src_tok, src_route));
  return PNV_OK;
}

// Built-in scratch for pnv_dispatch_plan_noalloc: per-chunk expert totals, chunks * E ints, at most
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

constexpr int kFinThreads = 128;

__global__ void __launch_bounds__(kFinThreads)
finalize_kernel(const __nv_bfloat16* __restrict__ fused, const int* __restrict__ route_dest,
                const float* __restrict__ topk_w, __nv_bfloat16* __restrict__ out, int topk, int K) {
  pdl_wait();
  pdl_launch_dependents();
  const long long t = blockIdx.x;
  const int col = (blockIdx.y * kFinThreads + threadIdx.x) * 8;
  if (col >= K) return;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int k = 0; k < topk; ++k) {
    const int d = route_dest[t * topk + k];
    if (d < 0) continue;   // dropped routing: its row is never read
    float v[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(fused + (long long)d * K + col)), v);
    if (topk_w != nullptr) {
      const float w = __bfloat162float(__float2bfloat16_rn(topk_w[t * topk + k]));
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], __bfloat162float(__float2bfloat16_rn(__fmul_rn(v[j], w))));
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], v[j]);
    }
  }
  __nv_bfloat16 o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(acc[j]);
  *reinterpret_cast<uint4*>(out + t * K + col) = *reinterpret_cast<const uint4*>(o);
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

}  // namespace
}  // namespace pnv

using namespace pnv;

extern "C" int64_t pnv_dispatch_plan_scratch_ints(int64_t n_routes, int num_local_experts) {
  const int64_t chunks = (n_routes + kChunk - 1) / kChunk;
  return chunks > 1 ? chunks * num_local_experts : 0;
}

extern "C" int pnv_dispatch_plan(const void* topk_ids, int ids_are_int64, int64_t tokens, int topk, int first_expert,
                                 int num_local_experts, int cap, int32_t* counts, int32_t* route_dest,
                                 int32_t* src_tok, int32_t* src_route, int32_t* scratch, pnv_stream_t stream) {
  PNV_REQUIRE(num_local_experts >= 1 && num_local_experts <= 4096, "num_local_experts must be in [1, 4096], got %d",
              num_local_experts);
  PNV_REQUIRE(cap >= 1, "cap must be positive");
  PNV_REQUIRE((long long)num_local_experts * cap < (1LL << 31), "E * cap must fit int32");
  PNV_REQUIRE(tokens >= 0 && topk >= 1 && tokens * topk < (1LL << 31), "T * topk must fit int32");
  PNV_REQUIRE(counts && (tokens == 0 || (topk_ids && route_dest && src_tok && src_route)), "null pointer argument");
  const long long n = (long long)tokens * topk;
  cudaStream_t s = (cudaStream_t)stream;
  if (ids_are_int64)
    return run_plan(static_cast<const long long*>(topk_ids), n, topk, first_expert, num_local_experts, cap, counts,
                    route_dest, src_tok, src_route, scratch, s);
  return run_plan(static_cast<const int*>(topk_ids), n, topk, first_expert, num_local_experts, cap, counts, route_dest,
                  src_tok, src_route, scratch, s);
}

extern "C" int64_t pnv_dispatch_plan_noalloc_max_scratch_ints(void) { return kBuiltinScratchInts; }

extern "C" int pnv_dispatch_plan_noalloc(const void* topk_ids, int ids_are_int64, int64_t tokens, int topk,
                                         int first_expert, int num_local_experts, int cap, int32_t* counts,
                                         int32_t* route_dest, int32_t* src_tok, int32_t* src_route,
                                         pnv_stream_t stream) {
  PNV_REQUIRE(tokens >= 0 && topk >= 1 && num_local_experts >= 1, "bad token count, topk or expert count");
  const int64_t need = pnv_dispatch_plan_scratch_ints(tokens * topk, num_local_experts);
  PNV_REQUIRE(need <= kBuiltinScratchInts,
              "dispatch_plan_noalloc: %lld routings over %d local experts need %lld scratch ints, the built-in "
              "scratch holds %d; use pnv_dispatch_plan with a caller-provided buffer",
              (long long)(tokens * topk), num_local_experts, (long long)need, kBuiltinScratchInts);
  int* scratch = nullptr;
  if (int rc = builtin_scratch(&scratch)) return rc;
  // Nothing in the scratch has to start at zero: the tally pass writes every total of every chunk
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
  const int slabs = (k + kFinThreads * 8 - 1) / (kFinThreads * 8);
  PNV_CUDA(launch_pdl(finalize_kernel, dim3((unsigned)tokens, (unsigned)slabs), dim3(kFinThreads), 0,
                      (cudaStream_t)stream, pdl_enabled(), (const __nv_bfloat16*)fused, (const int*)route_dest,
                      topk_weights, (__nv_bfloat16*)out, topk, k));
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
