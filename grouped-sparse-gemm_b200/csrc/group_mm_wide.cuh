// group_mm, wide token tiles (64 to 256 tokens per tile): prefill-sized problems.
//
// Included by group_mm.cu inside namespace pnv::{anonymous}, after Params, TileWalk and the status codes.
//
// One kernel in two forms.
//   single CTA (kPair = false)  one CTA per SM multiplies 128 weight rows by TILE_N tokens per tile.
//   CTA pair   (kPair = true)   a cluster of two CTAs on neighbouring SMs multiplies 256 weight rows by
//                               TILE_N tokens with one tcgen05.mma.sp.cta_group::2 per 128-K block.  Each
//                               CTA loads its own 128 weight rows (with their metadata and scales) and HALF
//                               of the token rows into its own shared memory with ordinary TMA copies (no
//                               cluster multicast anywhere), and the tensor cores of both SMs read the two
//                               halves.  Against the single-CTA form that halves the activation bytes an SM
//                               has to pull from L2 per unit of math, which is what bounds these shapes.  Both
//                               CTAs' tile loads count their bytes on the first CTA's barrier (.cta_group::2
//                               tiled loads), the second CTA's small bulk copies are relayed by a remote arrive.
//
// Tail tiles.  The last token tile of an expert is often nearly empty (256 +- 16 rows per expert leave every other
// expert a second tile of a dozen rows).  When it holds at most 64 live rows - and the launch has the tensor map for
// it (K a multiple of 256, tiles of 128 tokens or more) - the tile runs 64 tokens wide: a quarter or half of the
// activation bytes, one scale row-atom, MMAs a quarter or half as long.  Every role derives the width from counts[].
// The pair kernel with 256-token tiles has a variant (kDblTails) that multiplies such a tile against two M units per
// work item (WideCfg::kTailDouble); the host picks it when experts hold few token tiles.
//
// 22 warps per CTA:
//   warp 0   tile producer: TMA copies of the compressed weights and of the activations
//   warp 1   side producer: bulk copies of the metadata, SFA and SFB atoms (they sit in global memory in
//            the shape tensor memory wants)
//   2 - 3    MMA issuers (of a pair: in the first CTA only), alternate tiles, each into its own accumulator
//            stage: per pipeline stage they wait for one barrier, issue the MMAs and commit.  With one
//            accumulator stage (256 tokens) there is one issuer.
//   4 - 5    copiers (one thread each; of a pair: in the first CTA only): tcgen05.cp of every stage's scale and
//            metadata atoms from shared memory into the stage's slot of a ring in tensor memory (warp 4 the weight
//            scales and the metadata, warp 5 the activation scales), then a tcgen05.commit that tells the issuers
//            the slot is filled.  The copies are asynchronous and off the issuers' instruction stream.  In the
//            second CTA of a pair warp 4 only relays "my copies have landed" to the first CTA.
//   6 - 21   epilogue, four groups of four warps (one warp per lane quarter); a tile's chunks of token
//            columns are dealt round-robin to the groups
//
// Barriers per pipeline stage s: full[s] (this CTA's copies landed; in a pair's first CTA it also counts the
// second CTA's tile loads), peer_full[s] (pair: the second CTA's bulk copies landed, relayed to the first), sf_full[s] (copier's commit -> issuers: scales and metadata are in tensor
// memory), empty[s] (issuer's tcgen05.commit, delivered to both CTAs of a pair -> producers).  Per accumulator
// stage: acc_full (commit, both CTAs), acc_empty (all epilogue warps of the CTA or pair -> issuers).  Every wait
// is bounded.

template <int TILE_N, int STAGE_K, bool kPair, bool kDblTails = false>
struct WideCfg {
  static_assert(TILE_N == 64 || TILE_N == 128 || TILE_N == 256, "wide tile widths: 64, 128, 256");
  static_assert(STAGE_K == 256 || STAGE_K == 512, "stage depths: 256, 512");
  static constexpr int kCtas = kPair ? 2 : 1;
  static constexpr int kEpilogueWarps = 16;
  static constexpr int kFirstEpilogueWarp = 6;
  static constexpr int kThreads = (kFirstEpilogueWarp + kEpilogueWarps) * 32;
  static constexpr int kAtoms = STAGE_K / 128;
  static constexpr int kARowBytes = STAGE_K / 4;
  static constexpr int kABytes = kTileM * kARowBytes;
  static constexpr uint32_t kASwizzle = STAGE_K == 512 ? 2 : 4;
  static constexpr int kBRows = TILE_N / kCtas;              // token rows this CTA loads
  static constexpr int kBBoxes = STAGE_K / 256;
  static constexpr int kBBoxBytes = kBRows * 128;
  static constexpr int kBBytes = kBBoxes * kBBoxBytes;
  static constexpr int kEAtoms = STAGE_K / 256;
  static constexpr int kEBytes = 2048 * kEAtoms;
  static constexpr int kSfaBytes = 512 * kAtoms;
  static constexpr int kSfbRowAtoms = TILE_N > 128 ? 2 : 1;  // every CTA holds the scales of all TILE_N tokens
  static constexpr int kSfbBytes = kSfaBytes * kSfbRowAtoms;
  // a pipeline stage in shared memory: [weights | activations | metadata | weight scales | activation scales]
  static constexpr int kStageBytes = kABytes + kBBytes + kEBytes + kSfaBytes + kSfbBytes;
  static constexpr int kOffA = 0;
  static constexpr int kOffB = kABytes;
  static constexpr int kOffE = kOffB + kBBytes;
  static constexpr int kOffSfa = kOffE + kEBytes;
  static constexpr int kOffSfb = kOffSfa + kSfaBytes;
  static constexpr int kTailN = 64;                          // width of a narrow tail tile
  static constexpr int kTailBRows = kTailN / kCtas;
  static constexpr int kTailBBoxBytes = kTailBRows * 128;
  static constexpr int kChunk = TILE_N >= 128 ? 32 : 16;     // token columns an epilogue group takes at a time
  static constexpr int kFusedOutBytes = 4 * 8192;            // fused epilogue: one 8 KiB exchange area per group
  static constexpr int kPlainWarpWords = 8 * 36;             // plain epilogue: 8 token pairs x 32 features (+ 4 words of padding) per warp
  static constexpr int kPlainOutBytes = kEpilogueWarps * kPlainWarpWords * 4;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kMaxStages = 12;
  static constexpr int kAccStages = TILE_N == 256 ? 1 : 2;
  // tensor-memory columns: accumulators below 256, then a ring of slots, one per pipeline stage, each holding
  // the stage's weight scales, activation scales and metadata
  static constexpr int kColSlots = 256;
  static constexpr int kSfbColsPerAtom = 4 * kSfbRowAtoms;
  static constexpr int kSlotSfb = 4 * kAtoms;                // column offsets inside a slot
  static constexpr int kSlotE = kSlotSfb + kSfbColsPerAtom * kAtoms;
  // Double tail items (CTA pairs, 256-token tiles).  A narrow tail tile costs a pipeline stage per
  // 256 K like any other tile although it moves half the bytes and a quarter of the math, so such a tile is
  // multiplied against TWO M units per work item: the stage then holds both units' weights, metadata and weight
  // scales next to the one 64-token activation box, and the item writes two 64-column accumulators.  Half as many
  // stages per tail tile, and the activation box is fetched once for two units.  The support costs every item a few
  // instructions in roles whose instruction streams bound the pipeline, so it is a kernel variant of its own
  // (kDblTails), which the host picks when experts hold few token tiles.  The layout of such a stage:
  static constexpr bool kTailDouble = kDblTails && kPair && TILE_N == 256;
  static constexpr int kDblOffA1 = kABytes;                              // second unit's weights
  static constexpr int kDblOffB = 2 * kABytes;
  static constexpr int kDblOffE = kDblOffB + kBBoxes * kTailBBoxBytes;   // metadata, unit after unit
  static constexpr int kDblOffSfa = kDblOffE + 2 * kEBytes;              // weight scales, unit after unit
  static constexpr int kDblOffSfb = kDblOffSfa + 2 * kSfaBytes;          // activation scales (one row atom)
  static constexpr int kDblBytes = kDblOffSfb + kSfaBytes;
  // ... and of its tensor-memory slot: [SFA unit 0 | SFA unit 1 | SFB | E unit 0 | E unit 1]
  static constexpr int kDblSlotSfa1 = 4 * kAtoms;
  static constexpr int kDblSlotSfb = 8 * kAtoms;
  static constexpr int kDblSlotE = kDblSlotSfb + 4 * kAtoms;
  static constexpr int kDblSlotE1 = kDblSlotE + 4 * kEAtoms;
  static constexpr int kDblSlotCols = kDblSlotE1 + 4 * kEAtoms;
  static constexpr int kSlotCols = kTailDouble ? (kDblSlotCols > kSlotE + 4 * kEAtoms ? kDblSlotCols : kSlotE + 4 * kEAtoms)
                                               : kSlotE + 4 * kEAtoms;
  static constexpr int kSlots = (kTmemCols - kColSlots) / kSlotCols;    // caps the pipeline depth
  static_assert(kStageBytes % 1024 == 0 && kOffB % 1024 == 0, "operand tiles must keep 1024-byte alignment");
  static_assert(kAccStages * TILE_N <= kColSlots && kSlots >= 2, "tensor-memory column map overflows");
  static_assert(!kTailDouble || (kDblBytes <= kStageBytes && kDblOffB % 1024 == 0 && 2 * kTailN <= TILE_N),
                "a double tail stage must fit the ordinary stage");
  // the barriers take the first half of the barrier block, the per-stage item kinds sit in the second
  static_assert(8 * (4 * kMaxStages + 2 * kAccStages) + 16 <= kBarrierBytes / 2 && 4 * kMaxStages <= kBarrierBytes / 2,
                "barrier block overflows");
};

// Developer build only (-DPNV_WIDE_PROFILE): per-CTA cycle counters of the roles' waits, 16 per CTA, in a buffer
// read back with pnv_debug_wide_profile.  Not compiled into the library otherwise.
#ifdef PNV_WIDE_PROFILE
__device__ long long g_wide_prof[296 * 16];
#define PNV_PROF_T() clock64()
#define PNV_PROF_ACC(var, t0) var += clock64() - (t0)
#define PNV_PROF_SET(slot, v) g_wide_prof[blockIdx.x * 16 + (slot)] = (v)
#else
#define PNV_PROF_T() 0ll
#define PNV_PROF_ACC(var, t0) ((void)(t0), (void)(var))
#define PNV_PROF_SET(slot, v) ((void)(v))
#endif

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint64_t pack_desc(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Work items of an expert with c token rows: one per (token tile, M unit) - except that, with double tail items, the
// narrow tail tile (at most 64 live rows) takes one item per TWO M units.  full = the items of the ordinary tiles.
template <int TILE_N>
__device__ __forceinline__ unsigned expert_items(int c, int n_mu, bool dbl_tails, unsigned& full) {
  const unsigned nt = (unsigned)ceil_div_i(c, TILE_N);
  const bool tail = dbl_tails && c > 0 && c - (int)(nt - 1u) * TILE_N <= 64;
  full = (unsigned)n_mu * (nt - (tail ? 1u : 0u));
  return full + (tail ? (unsigned)(n_mu + 1) >> 1 : 0u);
}

// Work items position `unit` of `n_units` will process: items unit, unit + n_units, ... of the list every role
// walks.  Warp-collective.
template <int TILE_N>
__device__ __forceinline__ int my_work_items(const int* cnt, int E, int n_mu, bool dbl_tails, int unit, int n_units, int lane) {
  long long sum = 0;
  for (int e = lane; e < E; e += 32) {
    unsigned full;
    sum += expert_items<TILE_N>(cnt[e], n_mu, dbl_tails, full);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  return (long long)unit < sum ? (int)((sum - unit + n_units - 1) / n_units) : 0;
}

// The work items of one unit (a CTA, or a CTA pair), in the order every role walks them: items unit, unit + units,
// ... of the (expert, token tile, M unit) order, so that units working at the same time share token rows through L2.
// next() moves to the following item and says whether there was one.
template <int TILE_N>
struct UnitTiles {
  int e, mu, nt;                 // the current item: expert, (first) M unit, token tile
  bool dbl;                      // ... a narrow tail tile against M units mu and mu + 1
  // 32-bit walk (the host bounds the tile count of a launch): next item index, first item of expert e_next.  The
  // item count of an expert is recomputed from its row count whenever it is needed (a few instructions per item)
  // rather than carried along in registers.
  const int* cnt;
  int E, n_mu, e_next, n_units;
  bool dbl_tails;
  unsigned w, base;
  __device__ void init(const int* s_counts, int E_, int n_mu_, bool dbl_tails_, int unit, int n_units_) {
    cnt = s_counts; E = E_; n_mu = n_mu_; e_next = 0; n_units = n_units_; dbl_tails = dbl_tails_;
    w = (unsigned)unit; base = 0; dbl = false;
  }
  __device__ bool next() {
    unsigned full, items = expert_items<TILE_N>(cnt[e_next], n_mu, dbl_tails, full);
    while (w - base >= items) {
      base += items;
      if (++e_next >= E) return false;
      items = expert_items<TILE_N>(cnt[e_next], n_mu, dbl_tails, full);
    }
    const unsigned local = w - base;
    if (local < full) {
      nt = (int)(local / (unsigned)n_mu);
      mu = (int)(local - (unsigned)nt * (unsigned)n_mu);
      dbl = false;
    } else {                      // (only with dbl_tails: otherwise full == items)
      nt = (cnt[e_next] - 1) / TILE_N;
      mu = 2 * (int)(local - full);
      dbl = true;
    }
    e = e_next;
    w += (unsigned)n_units;
    return true;
  }
};

// Does the tile at token offset n0 of an expert with cnt rows run as a narrow tail tile?
template <int TILE_N>
__device__ __forceinline__ bool narrow_tail(const Params& p, int cnt, int n0) {
  return TILE_N >= 128 && p.b_tail != 0 && cnt - n0 <= 64;
}

// tensor memory -> registers, kChunk (16 or 32) consecutive columns of this warp's lane quarter
template <int N>
__device__ __forceinline__ void tc_ld_cols(uint32_t taddr, uint32_t (&r)[N]);
template <>
__device__ __forceinline__ void tc_ld_cols<32>(uint32_t taddr, uint32_t (&r)[32]) { ptx::tc_ld_32x32(taddr, r); }
template <>
__device__ __forceinline__ void tc_ld_cols<16>(uint32_t taddr, uint32_t (&r)[16]) { ptx::tc_ld_32x16(taddr, r); }
template <>
__device__ __forceinline__ void tc_ld_cols<8>(uint32_t taddr, uint32_t (&r)[8]) { ptx::tc_ld_32x8(taddr, r); }

template <int TILE_N, int STAGE_K, bool kFused, bool kPair, bool kDblTails>
__global__ void __launch_bounds__((6 + 16) * 32, 1)
group_mm_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_b_tail, const Params p) {
  using C = WideCfg<TILE_N, STAGE_K, kPair, kDblTails>;
  using Tiles = UnitTiles<TILE_N>;
  constexpr int kCtas = C::kCtas;
  constexpr int kChunk = C::kChunk;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint8_t* after_stages = stage_base + p.stages * C::kStageBytes;
  constexpr int kOutBytes = kFused ? C::kFusedOutBytes : C::kPlainOutBytes;
  uint8_t* s_out = after_stages;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(after_stages + kOutBytes);
  uint64_t* empty_bar = full_bar + C::kMaxStages;
  uint64_t* sf_full = empty_bar + C::kMaxStages;
  uint64_t* peer_full = sf_full + C::kMaxStages;
  uint64_t* acc_full = peer_full + C::kMaxStages;
  uint64_t* acc_empty = acc_full + C::kAccStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + C::kAccStages);
  // per pipeline stage: does it belong to a double tail item?  Written by the metadata producer before its
  // arrival on the stage's full barrier, read by the copiers after their wait on it.
  volatile int* s_kind = reinterpret_cast<volatile int*>(after_stages + kOutBytes + C::kBarrierBytes / 2);
  int* s_counts = reinterpret_cast<int*>(after_stages + kOutBytes + C::kBarrierBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // position of this CTA (or CTA pair) in the work list, and of this CTA inside its pair
  const uint32_t rank = kPair ? ptx::cluster_ctarank() : 0u;
  const int unit = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int n_units = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int n_mu = kPair ? (p.n_mt + 1) / 2 : p.n_mt;      // work items per token tile: M tiles, or pairs of them
  const bool dbl_tails = C::kTailDouble && p.b_tail != 0;  // narrow tail tiles take two M units per work item

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    ptx::prefetch_tensormap(&map_b_tail);
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(full_bar + s, 3);
      ptx::mbar_init(empty_bar + s, 1);
      ptx::mbar_init(sf_full + s, 2);
      ptx::mbar_init(peer_full + s, 1);
    }
    for (int a = 0; a < C::kAccStages; ++a) {
      ptx::mbar_init(acc_full + a, 1);
      ptx::mbar_init(acc_empty + a, C::kEpilogueWarps * kCtas);
    }
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc<kCtas>(tmem_slot, kTmemCols);
    ptx::tmem_relinquish<kCtas>();
  }
  // counts (and everything else the producer kernels wrote) may only be read after this point
  pdl_wait();
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < p.E; i += C::kThreads) s_counts[i] = max(0, min(p.counts[i], p.max_n));
  ptx::tc_fence_before();
  __syncthreads();
  if (kPair) ptx::cluster_sync();     // the partner's barriers are initialised before anything arrives on them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 2) {
    // =============================== producers ===============================
    // In each producer warp p.prod_lanes lanes work side by side, lane i on pipeline slots i, i + lanes, ...:
    // one thread needs several hundred cycles per (wait, expect, copy) sequence, while the same sequence
    // issued by several lanes in one go costs little more than once.  The loop carries its position (tile, K
    // stage, slot, turn) forward with additions only and recomputes addresses only when the tile changes.
    // The bulk-copy warp splits every stage between two lanes (metadata atoms; scale atoms), each with its
    // own expect-tx arrival, so a stage's full barrier counts three arrivals.
    const bool tile_role = warp == 0;
    const int slot_lane = tile_role ? lane : lane >> 1;     // which of the side-by-side pipeline slots
    const int part = lane & 1;                              // bulk-copy warp: 0 metadata, 1 scales
    if (slot_lane < p.prod_lanes) {
      Tiles tiles;
      tiles.init(s_counts, p.E, n_mu, dbl_tails, unit, n_units);
      bool ok = true;
      int n = 0, ks = slot_lane, stage = slot_lane, cur_n = -1;     // prod_lanes <= stages (host)
      uint32_t turn = 0;
      int e = 0, mt = 0, mt1 = 0, n0 = 0, sfb_row_atoms = 1;
      bool tail = false, dbl = false;
      const uint8_t *e_base = nullptr, *sfa_base = nullptr, *sfb_base = nullptr;
      long long pf_wait = 0;
      while (ok) {
        while (ks >= p.k_stages) { ks -= p.k_stages; ++n; }
        if (n != cur_n) {                                  // a new tile: where it is, and its operand bases
          bool any = true;
          while (cur_n < n && (any = tiles.next())) ++cur_n;
          if (!any) break;
          e = tiles.e;
          n0 = tiles.nt * TILE_N;
          // the second CTA of a pair takes the odd M tile; past the last tile it re-reads the last one (its
          // results are never stored), so every copy stays inside the expert's operands
          mt = kPair ? min(2 * tiles.mu + (int)rank, p.n_mt - 1) : tiles.mu;
          tail = narrow_tail<TILE_N>(p, s_counts[e], n0);
          // a double tail item: the second M unit's tile (again clamped: past the last unit its results are dropped)
          dbl = C::kTailDouble && tiles.dbl;
          mt1 = dbl ? min(2 * (tiles.mu + 1) + (int)rank, p.n_mt - 1) : mt;
          if (!tile_role) {
            sfb_base = p.sfb + (((long long)e * p.sfb_rt + (n0 >> 7)) * p.n_kt) * 512;
            sfb_row_atoms = (TILE_N > 128 && !tail) ? min(2, p.sfb_rt - (n0 >> 7)) : 1;
            e_base = p.e_meta + (((long long)e * p.e_k_atoms) * p.e_m_atoms + mt) * 2048;
            sfa_base = p.sfa + (((long long)e * p.n_mt + mt) * p.n_kt) * 512;
          }
        }
        const int k_atoms = min(C::kAtoms, p.n_kt - ks * C::kAtoms);
        const int b_boxes = (k_atoms + 1) / 2;
        const int e_atoms = (k_atoms + 1) / 2;
        const uint32_t sf_bytes = 512u * k_atoms;
        uint8_t* st = stage_base + stage * C::kStageBytes;
        const long long tp0 = PNV_PROF_T();
        if (!ptx::mbar_wait(empty_bar + stage, turn ^ 1u)) {
          atomicExch(&g_status, tile_role ? kProducerEmptyTimeout : kSideProducerTimeout);
          ok = false;
          break;
        }
        PNV_PROF_ACC(pf_wait, tp0);                             // waiting for a free stage
        if (tile_role) {
          // with the 4-D activation map one copy fetches all of the stage's 256-K chunks (a box past the
          // last chunk is zero-filled and still counts its full size)
          const int nb = n0 + (int)rank * (tail ? C::kTailBRows : C::kBRows);      // this CTA's share of the token rows
          const uint32_t tile_bytes = (dbl ? 2 * C::kABytes : C::kABytes) +
                                      (p.b_4d ? C::kBBoxes : b_boxes) * (tail ? C::kTailBBoxBytes : C::kBBoxBytes);
          if (kPair) {
            // The tiles of BOTH CTAs are counted on the first CTA's barrier (the second CTA's loads name it as
            // theirs: .cta_group::2), so nothing has to relay "the big copies have landed" across the pair; the
            // first CTA expects both CTAs' bytes (the boxes are the same size), the second only arrives.
            if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar + stage, 2 * tile_bytes);
            else ptx::mbar_arrive(full_bar + stage);
            ptx::tma_load_3d_pair(st + C::kOffA, &map_a, full_bar + stage, 0, ks * C::kARowBytes, mt * kTileM, e);
            if (dbl) {              // both units' weights, then the one narrow activation box
              ptx::tma_load_3d_pair(st + C::kDblOffA1, &map_a, full_bar + stage, 0, ks * C::kARowBytes, mt1 * kTileM, e);
              ptx::tma_load_4d_pair(st + C::kDblOffB, &map_b_tail, full_bar + stage, 0, 0, nb, ks * C::kBBoxes, e);
            } else if (tail) {      // (only with the 4-D maps)
              ptx::tma_load_4d_pair(st + C::kOffB, &map_b_tail, full_bar + stage, 0, 0, nb, ks * C::kBBoxes, e);
            } else if (p.b_4d) {
              ptx::tma_load_4d_pair(st + C::kOffB, &map_b, full_bar + stage, 0, 0, nb, ks * C::kBBoxes, e);
            } else {
              for (int b = 0; b < b_boxes; ++b)
                ptx::tma_load_3d_pair(st + C::kOffB + b * C::kBBoxBytes, &map_b, full_bar + stage, 0,
                                      ks * (STAGE_K / 2) + b * 128, nb, e);
            }
          } else {
            ptx::mbar_arrive_expect_tx(full_bar + stage, tile_bytes);
            ptx::tma_load_3d(st + C::kOffA, &map_a, full_bar + stage, ks * C::kARowBytes, mt * kTileM, e);
            if (tail) {             // (only with the 4-D maps)
              ptx::tma_load_4d(st + C::kOffB, &map_b_tail, full_bar + stage, 0, nb, ks * C::kBBoxes, e);
            } else if (p.b_4d) {
              ptx::tma_load_4d(st + C::kOffB, &map_b, full_bar + stage, 0, nb, ks * C::kBBoxes, e);
            } else {
              for (int b = 0; b < b_boxes; ++b)
                ptx::tma_load_3d(st + C::kOffB + b * C::kBBoxBytes, &map_b, full_bar + stage,
                                 ks * (STAGE_K / 2) + b * 128, nb, e);
            }
          }
        } else if (part == 0) {
          if (C::kTailDouble) s_kind[stage] = dbl ? 1 : 0;
          ptx::mbar_arrive_expect_tx(full_bar + stage, (dbl ? 2 : 1) * e_atoms * 2048);
          for (int ea = 0; ea < e_atoms; ++ea) {
            const uint8_t* src = e_base + (long long)(ks * C::kEAtoms + ea) * p.e_m_atoms * 2048;
            if (dbl) {
              ptx::bulk_load(st + C::kDblOffE + ea * 2048, src, 2048, full_bar + stage);
              ptx::bulk_load(st + C::kDblOffE + C::kEBytes + ea * 2048, src + (mt1 - mt) * 2048, 2048, full_bar + stage);
            } else {
              ptx::bulk_load(st + C::kOffE + ea * 2048, src, 2048, full_bar + stage);
            }
          }
        } else if (dbl) {
          ptx::mbar_arrive_expect_tx(full_bar + stage, sf_bytes * 3);
          const uint8_t* src = sfa_base + ks * (C::kAtoms * 512);
          ptx::bulk_load(st + C::kDblOffSfa, src, sf_bytes, full_bar + stage);
          ptx::bulk_load(st + C::kDblOffSfa + C::kSfaBytes, src + (long long)(mt1 - mt) * p.n_kt * 512, sf_bytes, full_bar + stage);
          ptx::bulk_load(st + C::kDblOffSfb, sfb_base + (long long)(ks * C::kAtoms) * 512, sf_bytes, full_bar + stage);
        } else {
          ptx::mbar_arrive_expect_tx(full_bar + stage, sf_bytes * (1 + sfb_row_atoms));
          ptx::bulk_load(st + C::kOffSfa, sfa_base + ks * (C::kAtoms * 512), sf_bytes, full_bar + stage);
          for (int ra = 0; ra < sfb_row_atoms; ++ra)
            ptx::bulk_load(st + C::kOffSfb + ra * C::kSfaBytes,
                           sfb_base + ((long long)ra * p.n_kt + ks * C::kAtoms) * 512, sf_bytes, full_bar + stage);
        }
        ks += p.prod_lanes;
        stage += p.prod_lanes;
        if (stage >= p.stages) { stage -= p.stages; turn ^= 1u; }
      }
      if (threadIdx.x == 0) PNV_PROF_SET(0, pf_wait);
      if (!ok) {
        // give copies already in flight time to land before the CTA's shared memory is released
#pragma unroll 1
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 2 || warp == 3) {
    // =============================== MMA issuers ===============================
    // A tcgen05.mma holds its issuing thread for about as long as it executes, so whatever else that
    // thread does between two MMAs is time the tensor pipe idles.  Two issuers in two warps take alternate
    // tiles, each into its own accumulator stage; while one is between MMAs the other's are executing.
    // Every tile's MMAs still come from one thread, in K order.  The issuer does no copies: it counts its
    // tiles once and then only waits, issues and commits.
    constexpr int kIssuers = C::kAccStages == 2 ? 2 : 1;
    const int issuer = warp - 2;
    const int n_items = my_work_items<TILE_N>(s_counts, p.E, n_mu, dbl_tails, unit, n_units, lane);
    if (lane == 0 && issuer < kIssuers && rank == 0) {
      constexpr uint32_t idesc_full = ptx::mma_sp_nvf4_idesc(TILE_N, kTileM * kCtas);
      constexpr uint32_t idesc_tail = ptx::mma_sp_nvf4_idesc(C::kTailN, kTileM * kCtas);
      Tiles tiles;
      tiles.init(s_counts, p.E, n_mu, dbl_tails, unit, n_units);
      int stage = 0, acc = kIssuers == 2 ? issuer : 0;
      uint32_t phase = 0, acc_phase = 0, soff = 0;
      bool ok = true;
      // Pass over the stages of a tile the other issuer takes.  Each one is waited for, not just
      // counted: a parity wait only tells two consecutive phases of a barrier apart, so an issuer
      // must see every turn of every slot, or after a long tile it would take an old phase for its own.
      long long pf_skip = 0;
      auto skip_stages = [&](int n) {
        const long long tk0 = PNV_PROF_T();
#pragma unroll 1
        for (int i = 0; i < n && ok; ++i) {
          if (!ptx::mbar_wait(sf_full + stage, phase)) {
            atomicExch(&g_status, kMmaScaleTimeout);
            ok = false;
          }
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        soff = (uint32_t)stage * (C::kStageBytes >> 4);
        PNV_PROF_ACC(pf_skip, tk0);
      };
      if (kIssuers == 2 && issuer == 1 && n_items > 1) skip_stages(p.k_stages);
      // first-tile descriptors, split into the 32-bit halves: only the low half changes with the address
      const uint64_t d_a0 = ptx::smem_desc(ptx::smem_u32(stage_base) + C::kOffA, 8 * C::kARowBytes, 16, C::kASwizzle);
      const uint64_t d_b0 = ptx::smem_desc(ptx::smem_u32(stage_base) + C::kOffB, 1024, 16, 2);
      const uint32_t lo_a0 = (uint32_t)d_a0, hi_a = (uint32_t)(d_a0 >> 32);
      const uint32_t lo_b0 = (uint32_t)d_b0, hi_b = (uint32_t)(d_b0 >> 32);
      const uint32_t slots0 = tmem_base + C::kColSlots;
      const int last_atoms = p.n_kt - (p.k_stages - 1) * C::kAtoms;     // K-blocks of a tile's last stage
      const long long ti0 = PNV_PROF_T();
      long long pf_acc = 0, pf_slot = 0, pf_issue = 0, pf_loop = 0;
      for (int item = kIssuers == 2 ? issuer : 0; item < n_items && ok; item += kIssuers) {
        // a 64-wide tile's scales sit 0 or 2 columns into the 128-row atom (even offsets only: the MMA
        // faults on an odd scale column); wider tiles start at column 0 and need no tile coordinates
        uint32_t sfb_off = 0;
        uint32_t idesc = idesc_full, bbox16 = C::kBBoxBytes >> 4;
        bool dbl = false;
        if (TILE_N < 128 || p.b_tail != 0) {
          // (two issuers: each walks every tile and uses every other one)
          bool any = true;
          for (int s = item < kIssuers ? item + 1 : kIssuers; s > 0 && any; --s) any = tiles.next();
          if (!any) break;
          if (TILE_N < 128) sfb_off = ((tiles.nt * TILE_N) & 127) >> 5;
          if (narrow_tail<TILE_N>(p, s_counts[tiles.e], tiles.nt * TILE_N)) {
            idesc = idesc_tail;
            bbox16 = C::kTailBBoxBytes >> 4;
            dbl = C::kTailDouble && tiles.dbl;
          }
        }
        const long long ta0 = PNV_PROF_T();
        if (!ptx::mbar_wait(acc_empty + acc, acc_phase ^ 1)) {
          atomicExch(&g_status, kMmaAccTimeout);
          ok = false;
          break;
        }
        PNV_PROF_ACC(pf_acc, ta0);                              // waiting for a free accumulator
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TILE_N;
        // The K loop of one item, compiled twice (ordinary items; double tail items) and chosen per item: whatever
        // the issuing thread executes between two MMAs is time the tensor pipe waits for, so the loop of an ordinary
        // item carries nothing of the other kind.
        auto item_stages = [&](auto dbl_kind, auto full_kind) {
          constexpr bool kDbl = decltype(dbl_kind)::value;
          constexpr bool kFull = decltype(full_kind)::value;      // K is a whole number of stages: no short last stage
#pragma unroll 1
          for (int ks = 0; ks < p.k_stages; ++ks) {
            const int k_atoms = kFull ? C::kAtoms : ks + 1 == p.k_stages ? last_atoms : C::kAtoms;
            const long long ts0 = PNV_PROF_T();
            if (!ptx::mbar_wait(sf_full + stage, phase)) {
              atomicExch(&g_status, kMmaScaleTimeout);
              ok = false;
              break;
            }
            PNV_PROF_ACC(pf_slot, ts0);                           // waiting for a filled slot (own tiles)
            ptx::tc_fence_after();
            const long long tm0 = PNV_PROF_T();
            // descriptors of this stage: the precomputed ones of stage 0 plus the stage's offset in
            // 16-byte units (the address field is the low 14 bits, so a 32-bit add cannot carry out)
            const uint32_t la = lo_a0 + soff, lb = lo_b0 + soff;
            const uint32_t slot = slots0 + stage * C::kSlotCols;
            if constexpr (kDbl) {
              // a narrow tail tile against two M units: the units' weights sit kABytes apart, their accumulators
              // kTailN columns apart, and both read the one activation box and its scales
              const uint32_t lbd = lb + ((C::kDblOffB - C::kOffB) >> 4);
#pragma unroll
              for (int ka = 0; ka < C::kAtoms; ++ka) {
                if (ka < k_atoms) {
                  const uint64_t db = pack_desc(lbd + (ka >> 1) * (C::kTailBBoxBytes >> 4) + (ka & 1) * 4, hi_b);
                  const uint32_t sfb_d = slot + C::kDblSlotSfb + ka * 4;
                  ptx::tc_mma_sp_nvf4<kCtas>(d_tmem, pack_desc(la + ka * 2, hi_a), db, idesc_tail, (ks | ka) != 0 ? 1u : 0u,
                                             slot + ka * 4, sfb_d, slot + C::kDblSlotE + ka * 2);
                  ptx::tc_mma_sp_nvf4<kCtas>(d_tmem + C::kTailN, pack_desc(la + (C::kDblOffA1 >> 4) + ka * 2, hi_a), db,
                                             idesc_tail, (ks | ka) != 0 ? 1u : 0u, slot + C::kDblSlotSfa1 + ka * 4, sfb_d,
                                             slot + C::kDblSlotE1 + ka * 2);
                }
              }
            } else {
              const uint32_t sfb_cols = slot + C::kSlotSfb + sfb_off;
#pragma unroll
              for (int ka = 0; ka < C::kAtoms; ++ka)
                if (kFull || ka < k_atoms)
                  ptx::tc_mma_sp_nvf4<kCtas>(d_tmem, pack_desc(la + ka * 2, hi_a),
                                             pack_desc(lb + (ka >> 1) * bbox16 + (ka & 1) * 4, hi_b), idesc,
                                             ka != 0 ? 1u : ks != 0 ? 1u : 0u, slot + ka * 4,
                                             sfb_cols + ka * C::kSfbColsPerAtom, slot + C::kSlotE + ka * 2);
            }
            // shared-memory stage and tensor-memory slot reusable (in both CTAs of a pair) once these MMAs retire
            ptx::tc_commit_n<kCtas>(empty_bar + stage);
            PNV_PROF_ACC(pf_issue, tm0);                          // issuing MMAs + commit
            soff += C::kStageBytes >> 4;
            if (++stage == p.stages) { stage = 0; soff = 0; phase ^= 1; }
          }
        };
        if (C::kTailDouble && dbl) item_stages(std::true_type{}, std::false_type{});
        else if (last_atoms == C::kAtoms) item_stages(std::false_type{}, std::true_type{});
        else item_stages(std::false_type{}, std::false_type{});
        if (!ok) break;
        ptx::tc_commit_n<kCtas>(acc_full + acc);
        if (kIssuers == 2) {
          acc_phase ^= 1;                 // this issuer's accumulator stage comes round every own tile
          if (item + kIssuers < n_items) skip_stages(p.k_stages);
        } else if (++acc == C::kAccStages) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
      PNV_PROF_ACC(pf_loop, ti0);
      if (issuer == 0) {   // issuer 0's waits and work (it takes every other tile), its whole loop, stages of the CTA
        PNV_PROF_SET(1, pf_acc); PNV_PROF_SET(2, pf_slot); PNV_PROF_SET(3, pf_issue); PNV_PROF_SET(4, pf_loop);
        PNV_PROF_SET(5, (long long)n_items * p.k_stages); PNV_PROF_SET(14, pf_skip);
      }
    }
    __syncwarp();
  } else if (warp == 4 || warp == 5) {
    // =============================== copiers ===============================
    // Both copiers take every pipeline stage and split its atoms: copier 0 the weight scales and the metadata,
    // copier 1 the activation scales.  Each commits on the stage's sf_full barrier (two arrivals).  Without
    // double tail items the copiers do not walk the tiles: a narrow tail tile loads one activation-scale row atom
    // instead of two, and the copy of the other (whatever an older stage left there) lands in columns its
    // 64-token MMAs never read.
    const int copier = warp - 4;
    const int n_items = my_work_items<TILE_N>(s_counts, p.E, n_mu, dbl_tails, unit, n_units, lane);
    const long long n_stages = (long long)n_items * p.k_stages;
    if (lane == 0 && (rank == 0 || (kPair && copier == 0))) {
      // of a pair's second CTA only warp 4 works here: it tells the first CTA when each stage's copies have landed
      const bool relay = rank != 0;
      const uint64_t d_sfa0 = ptx::smem_desc(ptx::smem_u32(stage_base) + C::kOffSfa, 128, 0, 0);
      const uint64_t d_sfb0 = ptx::smem_desc(ptx::smem_u32(stage_base) + C::kOffSfb, 128, 0, 0);
      const uint64_t d_e0 = ptx::smem_desc(ptx::smem_u32(stage_base) + C::kOffE, 128, 0, 0);
      const uint32_t lo_sfa0 = (uint32_t)d_sfa0, lo_sfb0 = (uint32_t)d_sfb0, lo_e0 = (uint32_t)d_e0;
      const uint32_t hi = (uint32_t)(d_e0 >> 32);           // the three descriptors differ in the address only
      const uint32_t slots0 = tmem_base + C::kColSlots;
      const int last_atoms = p.n_kt - (p.k_stages - 1) * C::kAtoms;
      const bool whole_stages = last_atoms == C::kAtoms;
      int stage = 0, ks = 0;
      uint32_t phase = 0;
      long long pf_cwait = 0, pf_cissue = 0;
      bool dbl = false;       // a double tail item's stages are laid out differently: the producer says which they are
      const uint32_t lo_st0 = (uint32_t)ptx::smem_desc(ptx::smem_u32(stage_base), 128, 0, 0);

#pragma unroll 1
      for (long long g = 0; g < n_stages; ++g) {
        const long long tc0 = PNV_PROF_T();
        if (!ptx::mbar_wait(full_bar + stage, phase) || (kPair && !relay && !ptx::mbar_wait(peer_full + stage, phase))) {
          atomicExch(&g_status, kScaleLoaderTimeout);
          break;
        }
        PNV_PROF_ACC(pf_cwait, tc0);                            // waiting for landed copies
        if (relay) {
          ptx::mbar_arrive_cluster(peer_full + stage, 0);
        } else {
          if (C::kTailDouble && dbl_tails && ks == 0) dbl = s_kind[stage] != 0;
          ptx::tc_fence_after();
          const long long tc1 = PNV_PROF_T();
          // (compiled twice: K a whole number of stages, so that no copy needs a guard; or a short last stage)
          auto copy_stage = [&](auto full_kind) {
            constexpr bool kFull = decltype(full_kind)::value;
            const int k_atoms = kFull ? C::kAtoms : ks + 1 == p.k_stages ? last_atoms : C::kAtoms;
            const uint32_t soff = (uint32_t)stage * (C::kStageBytes >> 4);
            const uint32_t slot = slots0 + stage * C::kSlotCols;
            if (C::kTailDouble && dbl) {
              // double tail item: copier 0 both units' weight scales, copier 1 the activation scales and both
              // units' metadata
              const uint32_t lo = lo_st0 + soff;
              if (copier == 0) {
  #pragma unroll
                for (int u = 0; u < 2; ++u)
  #pragma unroll
                  for (int ka = 0; ka < C::kAtoms; ++ka)
                    if (kFull || ka < k_atoms)
                      ptx::tc_cp_32x128b_warpx4<kCtas>(slot + u * C::kDblSlotSfa1 + ka * 4,
                                                       pack_desc(lo + ((C::kDblOffSfa + u * C::kSfaBytes) >> 4) + ka * 32, hi));
              } else {
  #pragma unroll
                for (int ka = 0; ka < C::kAtoms; ++ka)
                  if (kFull || ka < k_atoms)
                    ptx::tc_cp_32x128b_warpx4<kCtas>(slot + C::kDblSlotSfb + ka * 4, pack_desc(lo + (C::kDblOffSfb >> 4) + ka * 32, hi));
  #pragma unroll
                for (int u = 0; u < 2; ++u)
  #pragma unroll
                  for (int ea = 0; ea < C::kEAtoms; ++ea)
                    if (kFull || 2 * ea < k_atoms)
                      ptx::tc_cp_128x128b<kCtas>(slot + C::kDblSlotE + u * (C::kDblSlotE1 - C::kDblSlotE) + ea * 4,
                                                 pack_desc(lo + ((C::kDblOffE + u * C::kEBytes) >> 4) + ea * 128, hi));
              }
            } else if (copier == 0) {
  #pragma unroll
              for (int ka = 0; ka < C::kAtoms; ++ka)
                if (kFull || ka < k_atoms) ptx::tc_cp_32x128b_warpx4<kCtas>(slot + ka * 4, pack_desc(lo_sfa0 + soff + ka * 32, hi));
  #pragma unroll
              for (int ea = 0; ea < C::kEAtoms; ++ea)
                if (kFull || 2 * ea < k_atoms) ptx::tc_cp_128x128b<kCtas>(slot + C::kSlotE + ea * 4, pack_desc(lo_e0 + soff + ea * 128, hi));
            } else {
  #pragma unroll
              for (int ka = 0; ka < C::kAtoms; ++ka) {
                if (kFull || ka < k_atoms) {
  #pragma unroll
                  for (int ra = 0; ra < C::kSfbRowAtoms; ++ra)
                    ptx::tc_cp_32x128b_warpx4<kCtas>(slot + C::kSlotSfb + ka * C::kSfbColsPerAtom + ra * 4,
                                                     pack_desc(lo_sfb0 + soff + ra * (C::kSfaBytes >> 4) + ka * 32, hi));
                }
              }
            }
          };
          if (whole_stages) copy_stage(std::true_type{});
          else copy_stage(std::false_type{});
          ptx::tc_commit_local<kCtas>(sf_full + stage);     // arrives once the copies above have completed
          PNV_PROF_ACC(pf_cissue, tc1);                           // issuing copies
        }
        if (++ks == p.k_stages) ks = 0;
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
      if (copier == 0 && !relay) { PNV_PROF_SET(6, pf_cwait); PNV_PROF_SET(7, pf_cissue); }
    }
    __syncwarp();
  } else {
    // =============================== epilogue ===============================
    const int group = (warp - C::kFirstEpilogueWarp) >> 2;   // chunks of kChunk token columns are dealt to the four groups in turn
    const int sub = warp & 3;                  // tensor-memory lane quarter this warp may read
    const int m_local = sub * 32 + lane;       // accumulator row (output feature) held by this thread
    uint8_t* gbuf = s_out + group * 8192;
    int acc = 0;
    uint32_t acc_phase = 0;
    int flip = 0;                              // fused epilogue: which of the two exchange areas the next chunk uses
    if (kFused) {
      // Benign fill of GEMM2's scale buffer: every byte the epilogues will not write (rows at or
      // past counts[e], K-block slop) becomes 0x38.  All CTAs share the lines; live slots are
      // skipped, so the fill never races with a quantized scale.
      const int KB = p.f_n / kSfBlock;
      const unsigned lines = (unsigned)p.E * p.sfb_rt * p.f_n_kt * 32u;   // < 2^27, checked by the host
      const uint32_t w4 = kBenignSf * 0x01010101u;
      constexpr unsigned kFillThreads = C::kEpilogueWarps * 32;
#pragma unroll 1
      for (unsigned c = blockIdx.x * kFillThreads + (threadIdx.x - C::kFirstEpilogueWarp * 32); c < lines; c += gridDim.x * kFillThreads) {
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
    // A warp hands its accumulator stage back as soon as it has read its last chunk of it (of a pair: to the
    // first CTA, where the issuers wait).
    auto release_acc = [&]() {
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (kPair && rank != 0) ptx::mbar_arrive_cluster(acc_empty + acc, 0);
        else ptx::mbar_arrive(acc_empty + acc);
      }
    };
    long long pf_ewait = 0, pf_ework = 0, pf_f0 = 0, pf_f1 = 0, pf_f2 = 0, pf_f3 = 0;
    Tiles tiles;
    tiles.init(s_counts, p.E, n_mu, dbl_tails, unit, n_units);
    while (tiles.next()) {
      // A double tail item holds two M units' 64-column accumulators side by side: epilogue groups 0-1 take the
      // first unit's two chunks, groups 2-3 the second unit's.
      const bool dbl = C::kTailDouble && tiles.dbl;
      const int e = tiles.e, mu = tiles.mu + (dbl ? group >> 1 : 0), nt = tiles.nt;
      const int chunk0 = dbl ? group & 1 : group;          // this group's first chunk of token columns
      const int cnt = s_counts[e];
      const int mt = kPair ? 2 * mu + (int)rank : mu;
      // the second CTA of the last pair of an odd tile count stores nothing, nor does anyone for a double item's
      // second unit past the last one
      const bool mt_valid = mt < p.n_mt;
      const float alpha = p.alphas[e];
      const int n0 = nt * TILE_N;
      const long long te0 = PNV_PROF_T();
      if (!ptx::mbar_wait(acc_full + acc, acc_phase)) {
        atomicExch(&g_status, kEpilogueTimeout);
        break;
      }
      PNV_PROF_ACC(pf_ewait, te0);                              // waiting for an accumulator
      const long long te1 = PNV_PROF_T();
      ptx::tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(sub * 32) << 16) + acc * TILE_N + (dbl ? (group >> 1) * C::kTailN : 0);
      bool released = false;
      if (!kFused) {
        // Plain epilogue.  A warp holds 32 features x kChunk tokens of the accumulator: it scales and rounds them to
        // bf16, hands the accumulator back, and then stores - when the output rows are 16-byte aligned, through a
        // warp-private transpose in shared memory (no barrier beyond the warp's own), else one token row at a time
        // straight from registers (64 contiguous bytes per instruction).  Rows at or past counts[e] are skipped.
        const int m = mt * kTileM + m_local;
        constexpr int kOwn = TILE_N / (4 * kChunk);       // chunks of a tile each group takes (1, or 2 for 256 tokens)
        const bool mine = mt_valid && m < p.M;
        const bool wide_rows = (p.M & 7) == 0;            // output rows are 16-byte aligned
        uint32_t* tbuf = reinterpret_cast<uint32_t*>(s_out) + (warp - C::kFirstEpilogueWarp) * C::kPlainWarpWords;
        // One chunk at a time: load, (after the warp's last chunk) hand the accumulator back, scale and round two
        // tokens to a register (cvt.rn.bf16x2.f32: first argument in the low half), store.  A chunk's stores are
        // issued and forgotten, so taking the first chunk all the way before loading the second delays the
        // hand-back by little, and the two chunks never sit in registers together (that spilled, and the spill
        // traffic to L2 was of the order of the output itself).
#pragma unroll
        for (int j = 0; j < kOwn; ++j) {
          const int c0 = (chunk0 + 4 * j) * kChunk;
          const int rows = cnt - (n0 + c0);               // live token rows from c0 on; the same for all lanes
          uint32_t pk[kChunk / 2];
          if (rows > 0) {
            uint32_t v[kChunk];
            tc_ld_cols<kChunk>(t_row + c0, v);
            ptx::tc_ld_wait();
#pragma unroll
            for (int i = 0; i < kChunk; i += 2) {
              const __nv_bfloat162 pr = __floats2bfloat162_rn(__fmul_rn(alpha, __uint_as_float(v[i])),
                                                             __fmul_rn(alpha, __uint_as_float(v[i + 1])));
              pk[i / 2] = *reinterpret_cast<const uint32_t*>(&pr);
            }
          }
          if (j == kOwn - 1) {                            // the issuers may reuse the accumulator while this warp stores
            release_acc();
            released = true;
          }
          if (rows <= 0) continue;
          if (wide_rows && p.out_parts.n > 0) {
            // Rows bound for other GPUs' buffers.  The four warps of the group (one lane quarter = 32 features
            // each) put their slices side by side in shared memory ([token pair][128 feature words], 16 tokens at a
            // time), so that a store instruction carries 256 contiguous bytes of an output row (16 lanes x 16
            // bytes, two rows per instruction) instead of 64: fewer, larger writes on the link.  Two group
            // barriers per pass; every warp of the group sees the same chunks, so they arrive together.
            uint32_t* gst = reinterpret_cast<uint32_t*>(s_out) + group * (4 * C::kPlainWarpWords);
            const int pr_row = ((warp - C::kFirstEpilogueWarp) & 3) * 2 + (lane >> 4), fg = lane & 15;
            const int m8 = mt * kTileM + fg * 8;
            const bool mine8 = mt_valid && m8 < p.M;
            const int first = (fg >> 2) & 1;             // which half of its 32 bytes a lane reads first (bank spread)
#pragma unroll
            for (int h = 0; h < kChunk / 16; ++h) {
              const int t0 = h * 16 + 2 * pr_row;
              __nv_bfloat16 *d0 = nullptr, *d1 = nullptr;
              if (mine8 && t0 < rows) {
                const long long src = (long long)e * p.max_n + (n0 + c0 + t0);
                const int r0 = p.row_map[src], r1 = t0 + 1 < rows ? p.row_map[src + 1] : -1;
                if (r0 >= 0) d0 = mapped_row(p, r0) + m8;
                if (r1 >= 0) d1 = mapped_row(p, r1) + m8;
              }
              named_bar_sync(1 + group, 128);
#pragma unroll
              for (int q = 0; q < 8; ++q) gst[q * 128 + sub * 32 + lane] = pk[h * 8 + q];
              named_bar_sync(1 + group, 128);
              const uint32_t* src = gst + pr_row * 128 + fg * 8;
              const uint4 x0 = *reinterpret_cast<const uint4*>(src + first * 4);
              const uint4 x1 = *reinterpret_cast<const uint4*>(src + (1 - first) * 4);
              const uint4 a = first ? x1 : x0, b = first ? x0 : x1;
              if (d0 != nullptr)
                *reinterpret_cast<uint4*>(d0) = make_uint4(__byte_perm(a.x, a.y, 0x5410), __byte_perm(a.z, a.w, 0x5410),
                                                           __byte_perm(b.x, b.y, 0x5410), __byte_perm(b.z, b.w, 0x5410));
              if (d1 != nullptr)
                *reinterpret_cast<uint4*>(d1) = make_uint4(__byte_perm(a.x, a.y, 0x7632), __byte_perm(a.z, a.w, 0x7632),
                                                           __byte_perm(b.x, b.y, 0x7632), __byte_perm(b.z, b.w, 0x7632));
            }
          } else if (wide_rows) {
            // 16 tokens at a time through a private corner of shared memory ([token pair][feature] words, rows
            // padded to 36 words so that neither side has bank conflicts): lane (k, f) = (lane / 4, lane % 4)
            // reads features 8 f .. 8 f + 7 of token pair k and stores 16 bytes per token, so one instruction
            // writes 64 contiguous bytes of each of eight output rows instead of 64 bytes of one.
            const int pr_row = lane >> 2, fg = lane & 3;
            const int m8 = mt * kTileM + sub * 32 + fg * 8;
            const bool mine8 = mt_valid && m8 < p.M;
#pragma unroll
            for (int h = 0; h < kChunk / 16; ++h) {
              // where this lane's two tokens go (nullptr: not stored), before the values take up registers
              const int t0 = h * 16 + 2 * pr_row;          // this lane's even token inside the chunk
              __nv_bfloat16 *d0 = nullptr, *d1 = nullptr;
              if (mine8 && t0 < rows) {
                const long long src = (long long)e * p.max_n + (n0 + c0 + t0);
                if (p.row_map == nullptr) {
                  d0 = p.out + src * p.M + m8;
                  if (t0 + 1 < rows) d1 = d0 + p.M;
                } else {
                  const int r0 = p.row_map[src], r1 = t0 + 1 < rows ? p.row_map[src + 1] : -1;
                  if (r0 >= 0) d0 = mapped_row(p, r0) + m8;
                  if (r1 >= 0) d1 = mapped_row(p, r1) + m8;
                }
              }
              __syncwarp();
#pragma unroll
              for (int q = 0; q < 8; ++q) tbuf[q * 36 + lane] = pk[h * 8 + q];
              __syncwarp();
              const uint4 a = *reinterpret_cast<const uint4*>(tbuf + pr_row * 36 + fg * 8);
              const uint4 b = *reinterpret_cast<const uint4*>(tbuf + pr_row * 36 + fg * 8 + 4);
              if (d0 != nullptr)
                *reinterpret_cast<uint4*>(d0) = make_uint4(__byte_perm(a.x, a.y, 0x5410), __byte_perm(a.z, a.w, 0x5410),
                                                           __byte_perm(b.x, b.y, 0x5410), __byte_perm(b.z, b.w, 0x5410));
              if (d1 != nullptr)
                *reinterpret_cast<uint4*>(d1) = make_uint4(__byte_perm(a.x, a.y, 0x7632), __byte_perm(a.z, a.w, 0x7632),
                                                           __byte_perm(b.x, b.y, 0x7632), __byte_perm(b.z, b.w, 0x7632));
            }
          } else if (p.row_map == nullptr) {
            const int live = mine ? min(kChunk, rows) : 0;
            const long long pitch = p.M;
            unsigned short* dst = reinterpret_cast<unsigned short*>(p.out + ((long long)e * p.max_n + n0 + c0) * pitch + m);
#pragma unroll
            for (int i = 0; i < kChunk; i += 2) {
              const uint32_t w = pk[i / 2];
              if (i < live) dst[(long long)i * pitch] = (unsigned short)(w & 0xFFFFu);
              if (i + 1 < live) dst[(long long)(i + 1) * pitch] = (unsigned short)(w >> 16);
            }
          } else {
            // lane i holds the output row of the chunk's token i (kChunk <= 32); -1 past the live rows
            const int to_lane = lane < rows ? p.row_map[(long long)e * p.max_n + n0 + c0 + lane] : -1;
#pragma unroll
            for (int i = 0; i < kChunk; i += 2) {
              const uint32_t w = pk[i / 2];
              const int to0 = __shfl_sync(0xffffffffu, to_lane, i), to1 = __shfl_sync(0xffffffffu, to_lane, i + 1);
              if (mine && to0 >= 0) reinterpret_cast<unsigned short*>(mapped_row(p, to0))[m] = (unsigned short)(w & 0xFFFFu);
              if (mine && to1 >= 0) reinterpret_cast<unsigned short*>(mapped_row(p, to1))[m] = (unsigned short)(w >> 16);
            }
          }
        }
      } else {
        // Fused epilogue.  The weight rows are interleaved in 64-row blocks (32 gate rows, then the 32
        // matching up rows), so of a warp pair (lane quarters 0-1 or 2-3) one warp holds the gates and the
        // other the ups of the same 32 output features: exactly one quantization block per token.  The
        // pair splits the chunk's tokens: the gate warp finishes the first half, the up warp the second.
        // Each parks the half its partner needs (bf16 pairs, [token pair][feature]; two areas used in turn, so
        // one barrier per chunk is enough) and computes the activation for its own tokens.  Everything after
        // that stays in registers, a feature per lane: the block amax is a warp-wide integer max of the bf16
        // magnitudes, lane t works out the scale of token t and hands the multiplier back by shuffle, every
        // lane rounds its feature to e2m1 (eight tokens' codes to a register), and three exchange steps
        // inside each group of eight lanes transpose token and feature, so that a lane ends up with one
        // aligned word of one token's codes.
        constexpr int kHalf = kChunk / 2;                    // tokens each warp of a pair finishes
        constexpr int kPk = kHalf / 2;                       // ... as bf16 pairs
        const bool is_up = (sub & 1) != 0;
        const int par = is_up ? 1 : 0;
        uint32_t* xbuf = reinterpret_cast<uint32_t*>(gbuf + (sub >> 1) * 4096);
        const int pair_bar = 1 + group * 2 + (sub >> 1);
        const float gs = p.f_gpe ? p.f_gscale[e] : p.f_gscale[0];
        const bool table = p.f_act.kind == PNV_ACT_SILU && p.f_act.silu_tab != nullptr;
        const int kb = mt * 2 + (sub >> 1);                  // 32-feature block of the N-wide output
        uint8_t* code_col = p.f_b_out + kb * 16 + (lane >> 3) * 4;
        const long long code_pitch = p.f_n / 2;
        // tensor memory -> registers for one chunk: the half this warp finishes stays (bf16 pairs, the even token
        // in the low half), the half its partner finishes is parked in shared memory; two loads, because the column
        // offsets differ between the gate and the up warp and the register indices must not
        auto load_park = [&](int c0, uint32_t* x_mine, uint32_t (&own)[kPk]) {
          uint32_t v_own[kHalf], v_oth[kHalf];
          tc_ld_cols<kHalf>(t_row + c0 + par * kHalf, v_own);
          tc_ld_cols<kHalf>(t_row + c0 + (1 - par) * kHalf, v_oth);
          ptx::tc_ld_wait();
#pragma unroll
          for (int k = 0; k < kPk; ++k) {
            const __nv_bfloat162 po = __floats2bfloat162_rn(__fmul_rn(alpha, __uint_as_float(v_oth[2 * k])),
                                                           __fmul_rn(alpha, __uint_as_float(v_oth[2 * k + 1])));
            x_mine[k * 32 + lane] = *reinterpret_cast<const uint32_t*>(&po);
            const __nv_bfloat162 pr = __floats2bfloat162_rn(__fmul_rn(alpha, __uint_as_float(v_own[2 * k])),
                                                           __fmul_rn(alpha, __uint_as_float(v_own[2 * k + 1])));
            own[k] = *reinterpret_cast<const uint32_t*>(&pr);
          }
        };
        // the gate warp's SiLU lookups for its own tokens (issued before the barrier, so they are in flight across it)
        auto gate_lookups = [&](const uint32_t (&own)[kPk], float (&sv)[kHalf]) {
#pragma unroll
          for (int k = 0; k < kPk; ++k) {
            sv[2 * k] = __uint_as_float((uint32_t)__ldg(p.f_act.silu_tab + (own[k] & 0xFFFFu)) << 16);
            sv[2 * k + 1] = __uint_as_float((uint32_t)__ldg(p.f_act.silu_tab + (own[k] >> 16)) << 16);
          }
        };
        // everything after the exchange for one chunk: activation, block scale, codes, stores
        auto finish = [&](int c0, const uint32_t (&own)[kPk], const uint32_t* x_other, float (&sv)[kHalf], bool have_sv) {
          const long long tf2 = PNV_PROF_T();
          uint32_t oth[kPk];
#pragma unroll
          for (int k = 0; k < kPk; ++k) oth[k] = x_other[k * 32 + lane];
          uint32_t yp[kPk];                        // results, bf16 pairs again
          if (table) {
            if (is_up || !have_sv) {
#pragma unroll
              for (int k = 0; k < kPk; ++k) {
                const uint32_t gk = is_up ? oth[k] : own[k];
                sv[2 * k] = __uint_as_float((uint32_t)__ldg(p.f_act.silu_tab + (gk & 0xFFFFu)) << 16);
                sv[2 * k + 1] = __uint_as_float((uint32_t)__ldg(p.f_act.silu_tab + (gk >> 16)) << 16);
              }
            }
#pragma unroll
            for (int k = 0; k < kPk; ++k) {
              const uint32_t u = is_up ? own[k] : oth[k];
              const __nv_bfloat162 pr = __floats2bfloat162_rn(__fmul_rn(sv[2 * k], bf16_lo(u)), __fmul_rn(sv[2 * k + 1], bf16_hi(u)));
              yp[k] = *reinterpret_cast<const uint32_t*>(&pr);
            }
          } else {
#pragma unroll
            for (int k = 0; k < kPk; ++k) {
              const uint32_t g = is_up ? oth[k] : own[k], u = is_up ? own[k] : oth[k];
              const __nv_bfloat162 pr = __floats2bfloat162_rn(gated_act(bf16_lo(g), bf16_lo(u), p.f_act),
                                                             gated_act(bf16_hi(g), bf16_hi(u), p.f_act));
              yp[k] = *reinterpret_cast<const uint32_t*>(&pr);
            }
          }
          PNV_PROF_ACC(pf_f2, tf2);                // partner's values in, activation
          const long long tf3 = PNV_PROF_T();
          // block amax of own token t, left in lane t: bf16 magnitudes order like their bit patterns (NaN, which
          // fmaxf would skip, counts as zero)
          uint32_t amax_bits = 0;
#pragma unroll
          for (int k = 0; k < kPk; ++k) {
            uint32_t lo = yp[k] & 0x7FFFu, hi = (yp[k] >> 16) & 0x7FFFu;
            lo = lo > 0x7F80u ? 0u : lo;
            hi = hi > 0x7F80u ? 0u : hi;
            const uint32_t mlo = __reduce_max_sync(0xffffffffu, lo), mhi = __reduce_max_sync(0xffffffffu, hi);
            amax_bits = lane == 2 * k ? mlo : amax_bits;
            amax_bits = lane == 2 * k + 1 ? mhi : amax_bits;
          }
          uint32_t sf_byte;
          float inv_mine;
          block_scale(__uint_as_float(amax_bits << 16), gs, sf_byte, inv_mine);
          // this lane's feature of every own token -> e2m1, token i of each eight in nibble i
          uint32_t codes[(kHalf + 7) / 8];
#pragma unroll
          for (int r = 0; r < (kHalf + 7) / 8; ++r) codes[r] = 0u;
#pragma unroll
          for (int k = 0; k < kPk; ++k) {
            const float i0 = __shfl_sync(0xffffffffu, inv_mine, 2 * k), i1 = __shfl_sync(0xffffffffu, inv_mine, 2 * k + 1);
            codes[k >> 2] |= cvt_e2m1x2(__fmul_rn(bf16_lo(yp[k]), i0), __fmul_rn(bf16_hi(yp[k]), i1)) << (8 * (k & 3));
          }
          // 8 x 8 nibble transpose inside each group of eight lanes: afterwards lane 8 g + j holds, for own token j
          // (and 8 + j), the codes of features 8 g .. 8 g + 7 in order - word g of that token's 16 bytes
#pragma unroll
          for (int r = 0; r < (kHalf + 7) / 8; ++r) {
            uint32_t x = codes[r], y;
            y = __shfl_xor_sync(0xffffffffu, x, 1);
            x = (lane & 1) ? ((x & 0xF0F0F0F0u) | ((y & 0xF0F0F0F0u) >> 4)) : ((x & 0x0F0F0F0Fu) | ((y & 0x0F0F0F0Fu) << 4));
            y = __shfl_xor_sync(0xffffffffu, x, 2);
            x = (lane & 2) ? ((x & 0xFF00FF00u) | ((y & 0xFF00FF00u) >> 8)) : ((x & 0x00FF00FFu) | ((y & 0x00FF00FFu) << 8));
            y = __shfl_xor_sync(0xffffffffu, x, 4);
            x = (lane & 4) ? ((x & 0xFFFF0000u) | (y >> 16)) : ((x & 0x0000FFFFu) | (y << 16));
            const int t = 8 * r + (lane & 7);                 // own token of this word
            const int n = n0 + c0 + par * kHalf + t;
            if (t < kHalf && n < cnt)
              *reinterpret_cast<uint32_t*>(code_col + ((long long)e * p.max_n + n) * code_pitch) = x;
          }
          {
            const int n = n0 + c0 + par * kHalf + lane;       // lane t holds the scale of own token t
            if (lane < kHalf && n < cnt) p.f_sfb_out[sf_offset(e, n, kb, p.sfb_rt, p.f_n_kt)] = (uint8_t)sf_byte;
          }
          PNV_PROF_ACC(pf_f3, tf3);                // amax, scale, quantize, transpose, store
        };
        if (TILE_N == 256) {
          // Two chunks per warp and one accumulator stage: both chunks leave tensor memory first (own halves in
          // registers, partner halves in the two exchange areas) and the accumulator goes back to the issuer
          // before any of the arithmetic.  Two pair barriers per tile: the partner has finished reading the
          // previous tile's areas; this tile's are filled.
          const int cA = chunk0 * kChunk, cB = cA + 4 * kChunk;
          const bool liveA = n0 + cA < cnt, liveB = n0 + cB < cnt;
          if (mt_valid && liveA) {
            const long long tf0 = PNV_PROF_T();
            uint32_t* area0 = xbuf;
            uint32_t* area1 = xbuf + 2 * kPk * 32;
            uint32_t ownA[kPk], ownB[kPk];
            float sv[kHalf];
            named_bar_sync(pair_bar, 64);
            load_park(cA, area0 + par * (kPk * 32), ownA);
            if (liveB) load_park(cB, area1 + par * (kPk * 32), ownB);
            release_acc();
            released = true;
            PNV_PROF_ACC(pf_f0, tf0);              // tensor-memory loads, packing, parking
            const long long tf1 = PNV_PROF_T();
            if (table && !is_up) gate_lookups(ownA, sv);
            named_bar_sync(pair_bar, 64);
            PNV_PROF_ACC(pf_f1, tf1);              // the pair barrier
            finish(cA, ownA, area0 + (1 - par) * (kPk * 32), sv, true);
            if (liveB) finish(cB, ownB, area1 + (1 - par) * (kPk * 32), sv, false);
          }
        } else {
#pragma unroll 1
          for (int c0 = group * kChunk; c0 < TILE_N && n0 + c0 < cnt; c0 += 4 * kChunk) {
            const long long tf0 = PNV_PROF_T();
            uint32_t* area = xbuf + flip * (2 * kPk * 32);
            flip ^= 1;
            uint32_t own[kPk];
            float sv[kHalf];
            if (!mt_valid) {                       // the same for every thread of the CTA: nothing to compute or store
              release_acc();
              released = true;
              break;
            }
            load_park(c0, area + par * (kPk * 32), own);
            if (c0 + 4 * kChunk >= TILE_N || n0 + c0 + 4 * kChunk >= cnt) { release_acc(); released = true; }
            PNV_PROF_ACC(pf_f0, tf0);              // tensor-memory loads, packing, parking
            const long long tf1 = PNV_PROF_T();
            if (table && !is_up) gate_lookups(own, sv);
            named_bar_sync(pair_bar, 64);
            PNV_PROF_ACC(pf_f1, tf1);              // the pair barrier
            finish(c0, own, area + (1 - par) * (kPk * 32), sv, true);
          }
        }
      }
      if (!released) release_acc();
      PNV_PROF_ACC(pf_ework, te1);                              // this group's share of the tile
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
    }
    if (group == 0 && sub == 0 && lane == 0) {
      PNV_PROF_SET(8, pf_ewait); PNV_PROF_SET(9, pf_ework);
      PNV_PROF_SET(10, pf_f0); PNV_PROF_SET(11, pf_f1); PNV_PROF_SET(12, pf_f2); PNV_PROF_SET(13, pf_f3);
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (kPair) ptx::cluster_sync();     // the partner has stopped reading this CTA's shared and tensor memory
  if (warp == 2) {
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc<kCtas>(tmem_base, kTmemCols);
  }
}
