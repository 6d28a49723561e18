// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[e][M,N] (=|+=) A[e] * B[e]^T          fp32 accumulation in TMEM
//
// Roles per CTA (224 threads):
//   warps 0, 6  TMA producers (alternate K blocks): stream 128xBLOCK_K A tiles and
//               B tiles through a multi-stage shared-memory ring, completion on
//               "full" mbarriers
//   warp 1      MMA issuer (one thread; only the leader CTA of a pair issues):
//               tcgen05.mma into one of two 256-column TMEM accumulators,
//               tcgen05.commit releases smem stages and publishes accumulators
//   warps 2-5   epilogue: tcgen05.ld (thread = output row), convert, stage in
//               128-byte-swizzled shared memory, TMA store / TMA reduce-add
//
// kCtaGroup == 1: one CTA owns a 128x256 output tile (UMMA M128 N256).
// kCtaGroup == 2: a 2-CTA cluster owns a 256x256 tile (UMMA M256 N256,
//                 cta_group::2); each CTA loads its 128 rows of A and its 128
//                 rows of B, so B is fetched once per pair without any
//                 multicast load.
//
// Operands may each be K-major ([rows, K], K contiguous) or MN-major
// ([K, rows], rows contiguous: the layout of a weight-gradient operand or of a
// [IN, OUT] weight read as B).  The layout only changes the TMA boxes and two
// descriptor fields, so it is a runtime parameter.
//
// The accumulator ping-pong lets the MMA of tile i+1 overlap the drain of tile
// i.  Tiles are handed out to the persistent CTAs/clusters by one of three
// schedules (template parameter kSched):
//   kSchedDense     (batch, tile_m, tile_n, k_slice) items, grouped raster order
//   kSchedCeForward (row block, vocabulary chunk) items, each a run of
//                   consecutive column tiles whose epilogue carries the running
//                   softmax statistics of its rows
//   kSchedGrouped   variable-length row groups (experts) found through a
//                   device-side offsets array
//   kSchedGroupedWgrad  the same row groups as the REDUCTION axis: one output
//                   matrix per group, (group, row chunk, tile) items that
//                   reduce-add into it
//
// Epilogues (template parameter kEpi) are listed at EpilogueKind.
#pragma once

#include "ptx.cuh"

namespace b200 {

constexpr int kBlockK = 64;       // bf16 elements per K block = one 128-byte swizzle row
constexpr int kUmmaK = 16;        // K of one tcgen05.mma for 16-bit inputs
constexpr int kTileMCta = 128;    // output rows per CTA (= TMEM lanes)
constexpr int kTileN = 256;       // output columns per tile (= UMMA N)
constexpr int kGemmThreads = 224;
constexpr int kProducerWarp1 = 6;  // second TMA producer (warp 0 is the first)
constexpr int kTmemCols = 512;    // two 256-column fp32 accumulators
constexpr int kEpiBufBytes = 4096;  // 32 rows x 128 B, one per epilogue warp per buffer
#ifndef B200_RASTER_GROUP_M
#define B200_RASTER_GROUP_M 8
#endif
constexpr int kRasterGroupM = B200_RASTER_GROUP_M;  // tile rows walked together so B panels stay in L2
constexpr int kSubtileBytes = 64 * kBlockK * 2;  // one 64(mn) x 64(k) MN-major box
constexpr int kMaxGroups = 192;   // groups a grouped launch can address (its tables share the SM with a 225 KiB ring)

enum EpilogueKind : int {
  kEpiF32Tma = 0,       // fp32 C through TMA: store, or reduce-add when p.reduce != 0
  kEpiBf16Tma = 1,      // bf16 C through TMA store
  kEpiBf16Rmw = 2,      // bf16 C += acc: read C, add in fp32, round once, write
  kEpiCeForward = 3,    // no C: per-row running (max, sum-exp) and the target's logit
  kEpiCeBackward = 4,   // bf16 C = scale * (exp(acc - lse[row]) - [col == target[row]]), padding = 0
  kEpiBf16Grouped = 5,  // bf16 C for ragged row groups, optional SiLU; rows past the group are not written
  // Ragged row groups, B = [gate | up] column blocks: C = silu(gate) * up (half as wide as
  // the product), and optionally the bf16 gate/up panel itself as a second output.
  kEpiBf16GroupedGlu = 6,
  // fp32 C through TMA store plus the same values rounded to bf16 into a second matrix
  // (the operand copy the next GEMM reads; replaces a separate fp32 -> bf16 convert pass).
  kEpiF32DualBf16 = 7,
  // Ragged row groups, backward of the activation fused into the input-gradient GEMM:
  // C = acc * silu'(saved) (p.act_silu == 2, saved [rows, n]) or, for SwiGLU (p.act_silu == 3,
  // saved = the [rows, 2, n] gate/up panel), C [rows, 2, n] = {acc * up * silu'(gate), acc * silu(gate)}.
  kEpiBf16GroupedActBwd = 8,
  // Ragged row groups whose results go straight to OTHER GPUs: every group's rows are stored
  // (plain 16-byte stores, 128 bytes per row and chunk) into the buffer of the rank the rows
  // came from, at the place that rank's own permutation expects them.  The expert GEMM and the
  // return leg of the expert-parallel exchange in one kernel: the transfer rides under the MMAs.
  kEpiBf16GroupedPeer = 9,
};

__host__ __device__ constexpr bool epi_is_grouped(int epi) {
  return epi == kEpiBf16Grouped || epi == kEpiBf16GroupedGlu || epi == kEpiBf16GroupedActBwd ||
         epi == kEpiBf16GroupedPeer;
}

constexpr int kMaxPeerRanks = 8;
struct PeerBuffers {
  uint16_t* ptr[kMaxPeerRanks];
};

enum ScheduleKind : int { kSchedDense = 0, kSchedCeForward = 1, kSchedGrouped = 2, kSchedGroupedWgrad = 3 };

__host__ __device__ constexpr bool sched_is_grouped(int sched) {
  return sched == kSchedGrouped || sched == kSchedGroupedWgrad;
}

// kWide (CTA pairs only): a 256 x 512 tile per pair -- ONE 512-column accumulator instead of two
// of 256, two UMMAs (N = 256 each) per K = 16 step, 48 KiB stages.  A third less operand traffic
// from L2 per FLOP (A is loaded once per 512 columns), at the price of the ping-pong: the next
// tile's MMAs wait for this tile's drain.  For deep reductions only (weight gradients).
template <int kCtaGroup, bool kWide = false>
struct GemmCfg {
  static_assert(!kWide || kCtaGroup == 2, "wide tiles are a CTA-pair configuration");
  static constexpr int kTileNCfg = kWide ? 2 * kTileN : kTileN;   // output columns per tile
  static constexpr int kBRowsCta = kTileNCfg / kCtaGroup;         // B rows this CTA loads
  static constexpr int kABytes = kTileMCta * kBlockK * 2;         // 16 KiB
  static constexpr int kBBytes = kBRowsCta * kBlockK * 2;         // 32 / 16 KiB
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (kCtaGroup == 1 || kWide) ? 4 : 6;   // 192 KiB of operand ring
  static constexpr int kAccumulators = kWide ? 1 : 2;             // of kTileNCfg TMEM columns each
  static constexpr int kTileM = kTileMCta * kCtaGroup;
  static constexpr int kEpiBytes = 4 * 2 * kEpiBufBytes;          // 32 KiB staging
  static constexpr int kNumBarriers = 2 * kStages + 4;
  static constexpr int kSmemBytes =
      kStages * kStageBytes + kEpiBytes + kNumBarriers * 8 + 16 + 1024 /* alignment slack */;
};

struct GemmParams {
  CUtensorMap map_a;   // K-major: {K, rows, batch} box {64, 128, 1}; MN-major: {rows, K, batch} box {64, 64, 1}
  CUtensorMap map_b;   // K-major: box {64, 256 / cta_group, 1}; MN-major: box {64, 64, 1}
  CUtensorMap map_c;   // {N, M, batch} box {32 (fp32) | 64 (bf16), 32, 1}, 128-byte swizzle
  int* status;         // device status word, 0 = ok
  uint16_t* c_bf16;    // direct-store epilogues (kEpiBf16Rmw, kEpiBf16Grouped)
  long long ldc;       // elements, direct-store epilogues
  long long batch_stride_c;
  int m, n;            // logical extents (bounds of the direct-store epilogues)
  int tiles_m, tiles_n, batch;
  int k_blocks;        // ceil(K / 64)
  int split_k;         // >= 1
  int kb_per_split;    // ceil(k_blocks / split_k); every split is non-empty
  int a_mn, b_mn;      // 1 = MN-major
  int reduce;          // kEpiF32Tma: 1 = reduce-add into C
  // ---- cross-entropy epilogues
  const int* targets;  // [m] class index per row
  float2* ce_partials; // kEpiCeForward: [ce_chunks][m] running (max, sum-exp) per vocabulary chunk
  float* ce_target_logit;  // kEpiCeForward: [m], written by the chunk that holds the target column
  const float* ce_lse; // kEpiCeBackward: [m] log-sum-exp per row
  float ce_scale;      // kEpiCeBackward: upstream gradient / rows
  int ce_classes;      // columns at or beyond this index are padding
  int ce_chunks;       // kSchedCeForward: vocabulary chunks per row block
  // ---- grouped (ragged) rows
  const int* group_offsets;  // [groups + 1] first row of each group
  const int* group_b_index;  // [groups] which B matrix group g multiplies; null = g itself
  int groups;
  int act_silu;        // kEpiBf16Grouped: 1 = apply x * sigmoid(x) before rounding;
                       // kEpiBf16GroupedActBwd: 2 = SiLU backward, 3 = SwiGLU backward
  const uint16_t* saved;   // kEpiBf16GroupedActBwd: what the forward kept ([rows, n] or [rows, 2, n])
  long long ld_saved;
  // ---- kEpiBf16GroupedPeer: group g's rows go to peer_out.ptr[group_dst_rank[g]], rows
  // group_dst_row[g] + (row - first row of g), row stride ldc; rows at or beyond peer_rows are
  // not written (device status 105)
  PeerBuffers peer_out;
  const int* group_dst_rank;
  const int* group_dst_row;
  long long peer_rows;
  // ---- kEpiBf16GroupedGlu (the reference's [rows, 2, ff] gate/up panel, gpu/ops/src/lib.rs:1149-1171)
  int glu_cols;        // ff: B's "up" block starts this many columns after its "gate" block; C is [rows, ff]
  CUtensorMap map_d;   // optional second output, the bf16 panel {2 * ff, rows, 1}, box {64, 32, 1};
                       // kEpiF32DualBf16: the bf16 copy of C, {N, M, batch}, box {64, 32, 1};
                       // kEpiBf16Grouped: C before the activation, {N, rows, 1}, box {64, 32, 1}
  uint16_t* d_bf16;    // panel base (null = panel not written)
  long long ldd;       // panel row stride, elements
  // ---- dynamic tile scheduling (CTA pairs): [0] next work item, [1] clusters that have
  // finished fetching; both are zero between launches.  Null = static round-robin.
  int* sched_counter;
};

constexpr int kSchedRing = 16;   // items in flight per cluster are far fewer (stages + accumulators + 2)

struct Tile {
  int batch;       // index into the batch / expert dimension of B (and of A, C when dense)
  int m0;          // first output row of the CLUSTER's tile
  int m_end;       // rows at or beyond this are outside the tile's group (grouped schedule)
  int tile_n;
  int kb_begin, kb_count;
  int k0;          // first element of the tile's walk along K (kb_begin * 64 except in kSchedGroupedWgrad)
  int k_tail;      // elements of the walk's last K block that belong to it (64 = all of them)
  int first, last;  // position inside a kSchedCeForward run
  int group, group_row0;   // kSchedGrouped: the tile's group and that group's first row
};

// Iterates the tiles of one CTA/cluster.  All three roles run the same
// iterator, so they agree on the order without talking to each other.
template <int kSched, int kTileM>
struct TileWalk {
  const GemmParams& p;
  const int* group_tile_start;   // shared memory, kSchedGrouped: [groups + 1] first m-tile of each group
  int item, inner, step;
  // Dynamic scheduling: the cluster's items arrive through a ring in shared memory,
  // one 64-bit word (sequence number + 1, item or -1) per item, written by the
  // scheduler warp; every role polls the same sequence, so they still agree.
  const volatile unsigned long long* ring;   // null = static round-robin
  uint32_t seq;
  volatile int* abort_flag;

  __device__ TileWalk(const GemmParams& p_, const int* gts, int cluster_id, int num_clusters,
                      const volatile unsigned long long* ring_ = nullptr, volatile int* abort_ = nullptr)
      : p(p_), group_tile_start(gts), item(cluster_id), inner(0), step(num_clusters), ring(ring_), seq(0),
        abort_flag(abort_) {
    if (ring) item = fetch();
  }

  // Item number `seq` of this cluster, or -1 when the work has run out (or the wait did).
  __device__ int fetch() const {
    const volatile unsigned long long* slot = ring + (seq & (kSchedRing - 1));
    uint64_t start = 0;
    for (uint32_t spin = 1;; ++spin) {
      const unsigned long long w = *slot;
      if (static_cast<uint32_t>(w >> 32) == seq + 1u) return static_cast<int>(static_cast<uint32_t>(w));
      if ((spin & 0xff) == 0) {
        if (*abort_flag) return -1;
        const uint64_t now = global_timer_ns();
        if (start == 0) {
          start = now;
        } else if (now - start > kWaitLimitNs) {
          *abort_flag = 1;
          atomicCAS(p.status, 0, kDevTimeoutSchedule);
          return -1;
        }
      }
    }
  }

  __device__ int total_items() const {
    if constexpr (kSched == kSchedDense) return p.batch * p.tiles_m * p.tiles_n * p.split_k;
    else if constexpr (kSched == kSchedCeForward) return p.tiles_m * p.ce_chunks;
    else if constexpr (kSched == kSchedGrouped) return group_tile_start[p.groups] * p.tiles_n;
    else return group_tile_start[p.groups] * p.tiles_m * p.tiles_n;
  }

  __device__ bool get(Tile& t) const {
    if (item < 0 || item >= total_items()) return false;
    t.first = 1;
    t.last = 1;
    t.kb_begin = 0;
    t.kb_count = p.k_blocks;
    t.k0 = 0;
    t.k_tail = kBlockK;
    t.m_end = p.m;
    if constexpr (kSched == kSchedDense) {
      int split = item % p.split_k;
      int r = item / p.split_k;
      int tiles = p.tiles_m * p.tiles_n;
      t.batch = r / tiles;
      r -= t.batch * tiles;
      int per_group = kRasterGroupM * p.tiles_n;
      int group = r / per_group;
      int first_m = group * kRasterGroupM;
      int group_rows = min(p.tiles_m - first_m, kRasterGroupM);
      int in_group = r - group * per_group;
      t.m0 = (first_m + in_group % group_rows) * kTileM;
      t.tile_n = in_group / group_rows;
      t.kb_begin = split * p.kb_per_split;
      t.kb_count = min(p.kb_per_split, p.k_blocks - t.kb_begin);
      t.k0 = t.kb_begin * kBlockK;
    } else if constexpr (kSched == kSchedCeForward) {
      // Row blocks vary fastest, so the clusters running side by side walk the
      // same vocabulary chunk (shared W tiles in L2) on different rows.
      int chunk = item / p.tiles_m;
      int row_block = item - chunk * p.tiles_m;
      int base = p.tiles_n / p.ce_chunks, rem = p.tiles_n % p.ce_chunks;
      int first_tile = chunk * base + min(chunk, rem);
      int count = base + (chunk < rem ? 1 : 0);
      t.batch = 0;
      t.m0 = row_block * kTileM;
      t.tile_n = first_tile + inner;
      t.first = inner == 0;
      t.last = inner == count - 1;
    } else if constexpr (kSched == kSchedGrouped) {
      // item -> (m-tile over all groups, n-tile) with n fastest: the clusters running
      // side by side then cover a couple of dozen consecutive m-tiles (one to three
      // experts) times all n-tiles, so every A tile is fetched from HBM once and the
      // few expert matrices in use stay in L2.
      int tm = item / p.tiles_n;
      int tn = item - tm * p.tiles_n;
      // largest g with group_tile_start[g] <= tm (empty groups share a start and are skipped)
      int lo = 0, hi = p.groups - 1;
      while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (group_tile_start[mid] <= tm) lo = mid; else hi = mid - 1;
      }
      while (lo + 1 < p.groups && group_tile_start[lo + 1] <= tm) ++lo;
      const int g = lo;
      const int* group_row_start = group_tile_start + kMaxGroups + 1;   // offsets, staged in shared memory
      t.batch = p.group_b_index ? p.group_b_index[g] : g;
      t.m0 = group_row_start[g] + (tm - group_tile_start[g]) * kTileM;
      t.m_end = group_row_start[g + 1];
      t.tile_n = tn;
      t.group = g;
      t.group_row0 = group_row_start[g];
    }
    if constexpr (kSched == kSchedGroupedWgrad) {
      // item -> (row chunk over all groups, output tile) with the tile fastest: the clusters
      // running side by side multiply the same few thousand rows into different tiles of one
      // group's output, so those rows come from HBM once.  A chunk is kb_per_split K blocks of
      // one group's rows, counted from the group's first row; only a group's last block can be
      // short, and the rows behind it belong to the next group (see the MMA issuer).
      const int tiles = p.tiles_m * p.tiles_n;
      const int chunk = item / tiles;
      const int tile = item - chunk * tiles;
      int lo = 0, hi = p.groups - 1;
      while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (group_tile_start[mid] <= chunk) lo = mid; else hi = mid - 1;
      }
      while (lo + 1 < p.groups && group_tile_start[lo + 1] <= chunk) ++lo;
      const int g = lo;
      const int* group_row_start = group_tile_start + kMaxGroups + 1;
      const int first_row = group_row_start[g] + (chunk - group_tile_start[g]) * p.kb_per_split * kBlockK;
      const int rows = min(group_row_start[g + 1] - first_row, p.kb_per_split * kBlockK);
      t.batch = p.group_b_index ? p.group_b_index[g] : g;
      t.m0 = (tile % p.tiles_m) * kTileM;
      t.tile_n = tile / p.tiles_m;
      t.kb_count = (rows + kBlockK - 1) / kBlockK;
      t.k0 = first_row;
      t.k_tail = rows - (t.kb_count - 1) * kBlockK;
    }
    return true;
  }

  __device__ void next(const Tile& t) {
    if constexpr (kSched == kSchedCeForward) {
      if (!t.last) { ++inner; return; }
      inner = 0;
    }
    if (ring) {
      ++seq;
      item = fetch();
    } else {
      item += step;
    }
  }
};

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int kCtaGroup, int kEpi, int kSched, bool kWide = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ GemmParams p) {
  static_assert(!kWide || (kEpi == kEpiF32Tma && kSched == kSchedDense), "wide tiles: plain fp32 GEMM only");
  using Cfg = GemmCfg<kCtaGroup, kWide>;
  constexpr int kTileNK = Cfg::kTileNCfg;        // this instantiation's tile width
  using Walk = TileWalk<kSched, Cfg::kTileM>;
  extern __shared__ uint8_t smem_raw[];
  // kSchedGrouped: [0, groups]: first m-tile of each group; [kMaxGroups + 1, ...]: first row of each group
  // kSchedGroupedWgrad: [0, groups]: first row chunk of each group; then the first rows likewise
  __shared__ int group_tile_start[sched_is_grouped(kSched) ? 2 * (kMaxGroups + 1) : 1];
  // Dynamic scheduling (CTA pairs): this CTA's copy of the cluster's item ring, and how many
  // items this CTA's first producer warp has started (what the scheduler warp paces itself by).
  __shared__ __align__(8) unsigned long long sched_ring[kSchedRing];
  __shared__ int sched_progress;
  const bool dynamic = kCtaGroup == 2 && p.sched_counter != nullptr;

  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;   // swizzle atoms need 1024-byte alignment
  uint8_t* smem = smem_raw + (base - raw_addr);

  const uint32_t ring = base;
  const uint32_t epi = ring + Cfg::kStages * Cfg::kStageBytes;
  const uint32_t bars = epi + Cfg::kEpiBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (Cfg::kStages + s); };
  auto tmem_full_bar = [&](int a) { return bars + 8u * (2 * Cfg::kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bars + 8u * (2 * Cfg::kStages + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + (bars - base) + 8 * Cfg::kNumBarriers);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = kCtaGroup == 2 ? cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / kCtaGroup;
  const int num_clusters = gridDim.x / kCtaGroup;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 4 * kCtaGroup);   // one arrival per epilogue warp per CTA
    }
    *abort_flag = 0;
    for (int i = 0; i < kSchedRing; ++i) sched_ring[i] = 0ull;
    sched_progress = 0;
    fence_mbar_init();
    prefetch_tensormap(&p.map_a);
    prefetch_tensormap(&p.map_b);
    if (kEpi == kEpiF32Tma || kEpi == kEpiF32DualBf16 || kEpi == kEpiBf16Tma || kEpi == kEpiCeBackward ||
        (epi_is_grouped(kEpi) && kEpi != kEpiBf16GroupedPeer))
      prefetch_tensormap(&p.map_c);
    if (kEpi == kEpiBf16GroupedGlu || kEpi == kEpiF32DualBf16 || (kEpi == kEpiBf16Grouped && p.d_bf16))
      prefetch_tensormap(&p.map_d);
  }
  if constexpr (sched_is_grouped(kSched)) {
    // Every CTA derives the same tile table from the offsets array.
    if (warp == 3) {
      for (int g = lane; g <= p.groups; g += 32) group_tile_start[kMaxGroups + 1 + g] = p.group_offsets[g];
      __syncwarp();
      if (lane == 0) {
        // rows per unit of the table: an output tile's rows, or a reduction chunk's
        const int unit = kSched == kSchedGrouped ? Cfg::kTileM : p.kb_per_split * kBlockK;
        int run = 0;
        for (int g = 0; g < p.groups; ++g) {
          group_tile_start[g] = run;
          int rows = group_tile_start[kMaxGroups + 2 + g] - group_tile_start[kMaxGroups + 1 + g];
          run += (max(rows, 0) + unit - 1) / unit;
        }
        group_tile_start[p.groups] = run;
      }
    }
  }
  if (warp == 2) {
    tmem_alloc<kCtaGroup>(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish<kCtaGroup>();
  }
  tcgen05_fence_before_sync();
  if constexpr (kCtaGroup == 2) cluster_sync(); else __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 || warp == kProducerWarp1) {
    // ------------------------------------------------------------ TMA producers
    // Two producer threads (in different warps) take alternate K blocks: one
    // thread cannot issue the 2-5 bulk-tensor copies of a K block as fast as
    // the tensor cores consume one.
    // The whole warp walks the loop (so that addresses, coordinates and barrier
    // phases stay warp-uniform and live in uniform registers); one elected lane
    // issues the copies.
    {
      const uint32_t which = warp == 0 ? 0u : 1u;
      uint32_t g = 0;   // K blocks seen so far, over all of this CTA's tiles
      bool ok = true;
      Walk walk(p, group_tile_start, cluster_id, num_clusters, dynamic ? sched_ring : nullptr, abort_flag);
      Tile t;
      for (; ok && walk.get(t); walk.next(t)) {
        if (dynamic && which == 0 && cta_rank == 1 && lane == 0 && (kSched != kSchedCeForward || t.first))
          *reinterpret_cast<volatile int*>(&sched_progress) = static_cast<int>(walk.seq) + 1;
        const int m0 = t.m0 + static_cast<int>(cta_rank) * kTileMCta;
        // kEpiBf16GroupedGlu (CTA pairs only): the leader loads 128 "gate" columns of B, its
        // peer the 128 "up" columns glu_cols further on, so the accumulator holds gate in
        // columns 0-127 and the matching up values in columns 128-255.
        const int n0 = kEpi == kEpiBf16GroupedGlu
                           ? t.tile_n * (kTileN / 2) + static_cast<int>(cta_rank) * p.glu_cols
                           : t.tile_n * kTileNK + static_cast<int>(cta_rank) * (kCtaGroup == 2 ? kTileN / 2 : 0);
        const int a_batch = sched_is_grouped(kSched) ? 0 : t.batch;   // grouped A is one [rows, K] matrix
        const int b_batch = kSched == kSchedGroupedWgrad ? 0 : t.batch;   // and so is a weight gradient's B
        for (int kb = t.kb_begin; kb < t.kb_begin + t.kb_count; ++kb, ++g) {
          if ((g & 1u) != which) continue;
          const uint32_t stage = g % Cfg::kStages;
          const uint32_t phase = (g / Cfg::kStages) & 1u;
          ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1u, p.status, kDevTimeoutProducer, abort_flag));
          if (!ok) break;
          // Both CTAs of a pair complete their bytes on the leader's barrier.
          const uint32_t fb = kCtaGroup == 2 ? map_to_cta(full_bar(stage), 0) : full_bar(stage);
          const uint32_t a_dst = ring + stage * Cfg::kStageBytes;
          const uint32_t b_dst = a_dst + Cfg::kABytes;
          const int k0 = t.k0 + (kb - t.kb_begin) * kBlockK;
          if (elect_one()) {
            if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(stage), Cfg::kStageBytes * kCtaGroup);
            if (!p.a_mn) {
              tma_load_3d<kCtaGroup>(a_dst, &p.map_a, fb, k0, m0, a_batch);
            } else {
#pragma unroll
              for (int i = 0; i < kTileMCta / 64; ++i)
                tma_load_3d<kCtaGroup>(a_dst + i * kSubtileBytes, &p.map_a, fb, m0 + 64 * i, k0, a_batch);
            }
            // A wide tile is two 256-column halves: this CTA's 128 rows of B for each of them,
            // one after the other in the stage (the second UMMA of a K step reads the second).
#pragma unroll
            for (int half = 0; half < (kWide ? 2 : 1); ++half) {
              const int nh = n0 + half * kTileN;
              const uint32_t bh = b_dst + half * (Cfg::kBBytes / 2);
              constexpr int kRowsPerHalf = kWide ? kTileN / 2 : Cfg::kBRowsCta;
              if (!p.b_mn) {
                tma_load_3d<kCtaGroup>(bh, &p.map_b, fb, k0, nh, b_batch);
              } else {
#pragma unroll
                for (int i = 0; i < kRowsPerHalf / 64; ++i)
                  tma_load_3d<kCtaGroup>(bh + i * kSubtileBytes, &p.map_b, fb, nh + 64 * i, k0, b_batch);
              }
            }
          }
          __syncwarp();
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // Only the leader CTA of a pair issues.  As in the producers, the whole warp
    // runs the loop and one elected lane issues: the descriptors then live in
    // uniform registers, which is what tcgen05.mma takes its operands from, and
    // the issuing path from one MMA to the next stays short.
    if (cta_rank == 0) {
      const uint32_t idesc = make_idesc_bf16(Cfg::kTileM, kTileN, p.a_mn != 0, p.b_mn != 0);   // one UMMA: N = 256
      // K-major: LBO unused (encoded 1), next K=16 slice is 32 bytes along the swizzled row.
      // MN-major: LBO = one 64x64 subtile, next K=16 slice is 16 rows of 128 bytes.
      // The descriptors of stage 0 / slice 0 are built once; every other one differs
      // only in the start-address field (address >> 4, below bit 14).
      const uint64_t a_desc0 = make_smem_desc(ring, p.a_mn ? kSubtileBytes : 16, 1024);
      const uint64_t b_desc0 = make_smem_desc(ring + Cfg::kABytes, p.b_mn ? kSubtileBytes : 16, 1024);
      const uint64_t a_kadd = (p.a_mn ? 2048u : 32u) >> 4, b_kadd = (p.b_mn ? 2048u : 32u) >> 4;
      constexpr uint64_t kStageAdd = Cfg::kStageBytes >> 4;
      uint32_t stage = 0, phase = 0;
      int it = 0;
      bool ok = true;
      Walk walk(p, group_tile_start, cluster_id, num_clusters, dynamic ? sched_ring : nullptr, abort_flag);
      Tile t;
      for (; ok && walk.get(t); walk.next(t), ++it) {
        const int acc = kWide ? 0 : (it & 1);
        const uint32_t acc_phase = kWide ? (it & 1) : ((it >> 1) & 1);
        ok = __all_sync(0xffffffffu, mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, p.status, kDevTimeoutMma, abort_flag));
        if (!ok) break;
        tcgen05_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kTileNK;
        for (int kb = 0; kb < t.kb_count; ++kb) {
          ok = __all_sync(0xffffffffu, mbar_wait(full_bar(stage), phase, p.status, kDevTimeoutMma, abort_flag));
          if (!ok) break;
          tcgen05_fence_after_sync();
          if constexpr (kSched == kSchedGroupedWgrad) {
            // The last K block of a group runs past the group's end: the copy engine clips
            // only at the end of the whole array, so rows k_tail..63 of this stage hold the
            // NEXT group's rows -- or, behind the last group, whatever the buffer holds there,
            // which need not even be finite (so zeroing one operand would not do: 0 x NaN).
            // Those rows of A and of B are zeroed, in this CTA's stage and in the peer's, before
            // the tensor cores read them.  An MN-major stage keeps one K row per 128-byte line of
            // each 64-column subtile, and B's subtiles follow A's, so this is whole lines of
            // consecutive subtiles.
            if (kb == t.kb_count - 1 && t.k_tail < kBlockK) {
              constexpr int kSubtiles = (kTileMCta + Cfg::kBRowsCta) / 64;
              const uint32_t a_stage = ring + stage * Cfg::kStageBytes;
              const int lines = kBlockK - t.k_tail;                 // per subtile
              const int chunks = lines * 8;                          // 16-byte pieces per subtile
              for (int c = lane; c < chunks * kSubtiles * kCtaGroup; c += 32) {
                const int cta = c / (chunks * kSubtiles);
                const int rest = c - cta * chunks * kSubtiles;
                const int sub = rest / chunks;
                const uint32_t off = a_stage + sub * kSubtileBytes + t.k_tail * 128 + (rest - sub * chunks) * 16;
                if (cta == 0) st_shared_zero16(off);
                else st_shared_cluster_zero16(map_to_cta(off, 1));
              }
              fence_proxy_async_all();
              __syncwarp();
            }
          }
          const uint64_t da = a_desc0 + stage * kStageAdd;
          const uint64_t db = b_desc0 + stage * kStageAdd;
          if (elect_one()) {
            if constexpr (!kWide) {
              umma_bf16<kCtaGroup>(d_tmem, da, db, idesc, kb != 0 ? 1u : 0u);
#pragma unroll
              for (int k = 1; k < kBlockK / kUmmaK; ++k)
                umma_bf16<kCtaGroup>(d_tmem, da + k * a_kadd, db + k * b_kadd, idesc, 1u);
            } else {
              // two 256-column halves per K step: B's second half sits half a B stage further on
              constexpr uint64_t kHalfB = (Cfg::kBBytes / 2) >> 4;
#pragma unroll
              for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                const uint32_t accumulate = (kb != 0 || k != 0) ? 1u : 0u;
                umma_bf16<kCtaGroup>(d_tmem, da + k * a_kadd, db + k * b_kadd, idesc, accumulate);
                umma_bf16<kCtaGroup>(d_tmem + kTileN, da + k * a_kadd, db + kHalfB + k * b_kadd, idesc, accumulate);
              }
            }
            umma_commit<kCtaGroup>(empty_bar(stage));   // stage reusable once these MMAs retire
          }
          __syncwarp();
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok && elect_one()) umma_commit<kCtaGroup>(tmem_full_bar(acc));   // accumulator ready for the epilogue
        __syncwarp();
      }
    } else if (dynamic) {
      // ---------------------------------------------------------- tile scheduler
      // The second CTA's warp 1 has no MMAs to issue; one of its lanes hands the cluster
      // its work instead: it takes the next item from a counter in global memory and
      // writes it into both CTAs' rings, staying exactly one item ahead of the producers.
      // A cluster that becomes resident late (another kernel held its SMs) simply finds
      // less work left, where a fixed round-robin share would make it a second wave.
      if (lane == 0) {
        Walk counting(p, group_tile_start, 0, 1);
        const int total = counting.total_items();
        const uint32_t own_ring = smem_u32(sched_ring);
        const uint32_t leader_ring = map_to_cta(own_ring, 0);
        bool ok = true;
        for (uint32_t q = 0;; ++q) {
          uint64_t start = 0;
          for (uint32_t spin = 1;
               ok && q > static_cast<uint32_t>(*reinterpret_cast<volatile int*>(&sched_progress)); ++spin) {
            __nanosleep(64);
            if ((spin & 0x3f) == 0) {
              if (*abort_flag) { ok = false; break; }
              const uint64_t now = global_timer_ns();
              if (start == 0) {
                start = now;
              } else if (now - start > kWaitLimitNs) {
                *abort_flag = 1;
                atomicCAS(p.status, 0, kDevTimeoutSchedule);
                ok = false;
              }
            }
          }
          const int item = ok ? atomicAdd(p.sched_counter, 1) : total;
          const uint32_t v = item < total ? static_cast<uint32_t>(item) : 0xffffffffu;
          const unsigned long long word = (static_cast<unsigned long long>(q + 1u) << 32) | v;
          const uint32_t off = (q & (kSchedRing - 1)) * 8u;
          st_shared_u64(own_ring + off, word);
          st_shared_cluster_u64(leader_ring + off, word);
          if (v == 0xffffffffu) break;
        }
        // The last cluster to run out of work leaves the counters at zero for the next launch.
        __threadfence();
        if (atomicAdd(p.sched_counter + 1, 1) == num_clusters - 1) {
          atomicExch(p.sched_counter, 0);
          atomicExch(p.sched_counter + 1, 0);
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;                 // TMEM lanes this warp may read
    const uint32_t lane_base = quarter * 32u;
    const uint32_t my_epi = epi + (warp - 2) * 2 * kEpiBufBytes;
    uint32_t chunk_counter = 0;
    int it = 0;
    bool ok = true;
    // kEpiCeForward: running statistics of this thread's row over a chunk of the vocabulary.
    float run_max = -INFINITY, run_sum = 0.f, target_logit = 0.f;
    bool have_target = false;
    constexpr float kLog2e = 1.4426950408889634f;
    Walk walk(p, group_tile_start, cluster_id, num_clusters, dynamic ? sched_ring : nullptr, abort_flag);
    Tile t;
    for (; ok && walk.get(t); walk.next(t), ++it) {
      const int acc = kWide ? 0 : (it & 1);
      const uint32_t acc_phase = kWide ? (it & 1) : ((it >> 1) & 1);
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, p.status, kDevTimeoutEpilogue, abort_flag)) {
        ok = false;
        break;
      }
      tcgen05_fence_after_sync();
      const int row0 = t.m0 + static_cast<int>(cta_rank) * kTileMCta + lane_base;   // warp's first row
      const int col0 = t.tile_n * (kEpi == kEpiBf16GroupedGlu ? kTileN / 2 : kTileNK);
      const uint32_t t_acc = tmem_base + (lane_base << 16) + acc * kTileNK;

      auto release_accumulator = [&]() {
        tcgen05_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kCtaGroup == 2) mbar_arrive_cluster(map_to_cta(tmem_empty_bar(acc), 0));
          else mbar_arrive(tmem_empty_bar(acc));
        }
      };
      // Write 32 rows x 128 bytes (this thread's 8 x 16 bytes) into a staging
      // buffer with the 128-byte swizzle the C tensor map expects.
      auto stage_row = [&](uint32_t buf, const uint32_t* v) {
        const uint32_t row_addr = buf + lane * 128u;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t dst = row_addr + ((static_cast<uint32_t>(j) ^ (lane & 7u)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v[4 * j]),
                       "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                       : "memory");
        }
      };

      if constexpr (kEpi == kEpiF32Tma || kEpi == kEpiF32DualBf16) {
        constexpr int kChunks = kTileNK / 32;
        [[maybe_unused]] uint32_t packed[32];       // kEpiF32DualBf16: two fp32 chunks make one bf16 chunk
        constexpr int kStep = kEpi == kEpiF32DualBf16 ? 2 : 1;
#pragma unroll 1
        for (int c0 = 0; c0 < kChunks; c0 += kStep) {
#pragma unroll
        for (int h = 0; h < kStep; ++h) {
          const int c = c0 + h;
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c * 32, r);
          tmem_ld_wait();
          if (c == kChunks - 1) release_accumulator();
          const uint32_t buf = my_epi + (chunk_counter & 1u) * kEpiBufBytes;
          if (lane == 0) tma_wait_group_read<1>();   // the store that last read this buffer is done
          __syncwarp();
          stage_row(buf, r);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (kEpi == kEpiF32Tma && p.reduce) tma_reduce_add_3d(&p.map_c, buf, col0 + c * 32, row0, t.batch);
            else tma_store_3d(&p.map_c, buf, col0 + c * 32, row0, t.batch);
            tma_commit_group();
          }
          ++chunk_counter;
          if constexpr (kEpi == kEpiF32DualBf16) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              packed[h * 16 + j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            if (h == 1) {
              const uint32_t buf2 = my_epi + (chunk_counter & 1u) * kEpiBufBytes;
              if (lane == 0) tma_wait_group_read<1>();
              __syncwarp();
              stage_row(buf2, packed);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&p.map_d, buf2, col0 + (c - 1) * 32, row0, t.batch);
                tma_commit_group();
              }
              ++chunk_counter;
            }
          }
        }
        }
      } else if constexpr (kEpi == kEpiBf16Tma || kEpi == kEpiCeBackward || epi_is_grouped(kEpi)) {
        constexpr bool kGlu = kEpi == kEpiBf16GroupedGlu;
        constexpr int kChunks = (kGlu ? kTileN / 2 : kTileN) / 64;
        const int row = row0 + lane;
        // kEpiCeBackward: p = exp(logit - lse) computed as exp2(logit*log2e - lse*log2e).
        float neg_lse2 = 0.f;
        int target = -1;
        if constexpr (kEpi == kEpiCeBackward) {
          if (row < p.m) {
            neg_lse2 = log2f(fabsf(p.ce_scale)) - p.ce_lse[row] * kLog2e;   // sign applied below
            target = p.targets[row];
          }
        }
        // kEpiBf16Grouped: a warp whose 32 rows all belong to the group uses the
        // TMA store; a warp that straddles the group's end writes row by row.
        bool warp_inside = true;
        if constexpr (epi_is_grouped(kEpi)) warp_inside = row0 + 32 <= t.m_end;
        // Stage 32 rows x 64 bf16 columns and send them through `map` to (col, row0), or,
        // for a warp that straddles the end of its group, write this thread's row directly.
        auto put_chunk = [&](const CUtensorMap* map, uint16_t* base_ptr, long long ld, int col, int col_end,
                             const uint32_t* packed) {
          if constexpr (kEpi == kEpiBf16GroupedPeer) {
            // Through shared memory, so that eight lanes write one row's 128 bytes side by side
            // (four rows per store instruction) instead of every lane writing 16 bytes of a row
            // of its own: the stores cross NVLink, where the size of a write matters.
            const uint32_t buf = my_epi + (chunk_counter & 1u) * kEpiBufBytes;
            stage_row(buf, packed);
            __syncwarp();
            uint16_t* dst_base = p.peer_out.ptr[p.group_dst_rank[t.group]];
            const long long dst_row0 = static_cast<long long>(p.group_dst_row[t.group]) + (row0 - t.group_row0);
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int rr = it * 4 + (lane >> 3);
              const int j = lane & 7;
              uint32_t v0, v1, v2, v3;
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                           : "r"(buf + rr * 128u + ((static_cast<uint32_t>(j) ^ (rr & 7u)) << 4)));
              const long long dr = dst_row0 + rr;
              if (row0 + rr < t.m_end && col + 8 * j + 8 <= col_end) {
                if (dr < p.peer_rows) {
                  *reinterpret_cast<uint4*>(dst_base + dr * ld + col + 8 * j) = make_uint4(v0, v1, v2, v3);
                } else {
                  atomicCAS(p.status, 0, kDevInboxOverflow);
                }
              }
            }
            __syncwarp();
            ++chunk_counter;
            return;
          }
          if (warp_inside) {
            const uint32_t buf = my_epi + (chunk_counter & 1u) * kEpiBufBytes;
            if (lane == 0) tma_wait_group_read<1>();
            __syncwarp();
            stage_row(buf, packed);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(map, buf, col, row0, sched_is_grouped(kSched) ? 0 : t.batch);
              tma_commit_group();
            }
            ++chunk_counter;
          } else if (row < t.m_end) {
            uint16_t* crow = base_ptr + static_cast<long long>(row) * ld;
            if (col + 64 <= col_end) {
              uint4* ptr = reinterpret_cast<uint4*>(crow + col);
#pragma unroll
              for (int q = 0; q < 8; ++q)
                ptr[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
            } else {
              for (int j = 0; j < 64 && col + j < col_end; ++j)
                crow[col + j] = static_cast<uint16_t>((packed[j >> 1] >> ((j & 1) * 16)) & 0xffffu);
            }
          }
        };
#pragma unroll 1
        for (int c = 0; c < kChunks; ++c) {
          uint32_t packed[32];
          if constexpr (kGlu) {
            // gate in accumulator columns [c*64, +64), up 128 columns further on
            uint32_t pg[32], pu[32];
            const bool panel = p.d_bf16 != nullptr;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t g[32], u[32];
              tmem_ld_32x32(t_acc + c * 64 + h * 32, g);
              tmem_ld_32x32(t_acc + kTileN / 2 + c * 64 + h * 32, u);
              tmem_ld_wait();
              if (panel) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  pg[h * 16 + j] = pack_bf16x2(__uint_as_float(g[2 * j]), __uint_as_float(g[2 * j + 1]));
                  pu[h * 16 + j] = pack_bf16x2(__uint_as_float(u[2 * j]), __uint_as_float(u[2 * j + 1]));
                }
              }
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                // silu(g) * u with silu(g) = hg + hg * tanh(hg), hg = g / 2
                const float hg = 0.5f * __uint_as_float(g[j]);
                g[j] = __float_as_uint(fmaf(hg, fast_tanh(hg), hg) * __uint_as_float(u[j]));
              }
#pragma unroll
              for (int j = 0; j < 16; ++j)
                packed[h * 16 + j] = pack_bf16x2(__uint_as_float(g[2 * j]), __uint_as_float(g[2 * j + 1]));
            }
            if (c == kChunks - 1) release_accumulator();
            const int col = col0 + c * 64;
            put_chunk(&p.map_c, p.c_bf16, p.ldc, col, p.n, packed);
            // The panel's gate block ends where its up block starts, so a chunk of gate
            // columns must not run past it (the host requires ff % 64 == 0 with a panel).
            if (panel && col < p.glu_cols) {
              put_chunk(&p.map_d, p.d_bf16, p.ldd, col, p.glu_cols, pg);
              put_chunk(&p.map_d, p.d_bf16, p.ldd, p.glu_cols + col, 2 * p.glu_cols, pu);
            }
          } else {
          // kEpiBf16Grouped with a second output: the values before the activation, which the
          // activation's backward reads.
          [[maybe_unused]] uint32_t before[32];
          const bool keep_before = kEpi == kEpiBf16Grouped && p.d_bf16 != nullptr;
          // kEpiBf16GroupedActBwd: this row's 64 saved values (and, for SwiGLU, the 64 "up"
          // values n columns further on), requested before the accumulator is read.
          [[maybe_unused]] uint4 sg[8], su[8];
          [[maybe_unused]] uint32_t packed_up[32];
          if constexpr (kEpi == kEpiBf16GroupedActBwd) {
            const uint16_t* srow = p.saved + static_cast<long long>(row) * p.ld_saved + col0 + c * 64;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const bool ok = row < t.m_end && col0 + c * 64 + 8 * q + 8 <= p.n;
              sg[q] = ok ? *reinterpret_cast<const uint4*>(srow + 8 * q) : make_uint4(0u, 0u, 0u, 0u);
              if (p.act_silu == 3)
                su[q] = ok ? *reinterpret_cast<const uint4*>(srow + p.n + 8 * q) : make_uint4(0u, 0u, 0u, 0u);
            }
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld_32x32(t_acc + c * 64 + h * 32, r);
            tmem_ld_wait();
            if constexpr (kEpi == kEpiBf16GroupedActBwd) {
              const uint32_t* gw = reinterpret_cast<const uint32_t*>(sg) + h * 16;
              const uint32_t* uw = reinterpret_cast<const uint32_t*>(su) + h * 16;
              float up_grad[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const uint32_t gword = gw[j >> 1];
                const float g = __uint_as_float((j & 1) ? (gword & 0xffff0000u) : (gword << 16));
                // sigmoid(g) = (1 + tanh(g / 2)) / 2: one MUFU op; silu'(g) = s * (1 + g * (1 - s))
                const float sgm = fmaf(0.5f, fast_tanh(0.5f * g), 0.5f);
                const float dsilu = sgm * fmaf(g, 1.f - sgm, 1.f);
                const float dy = __uint_as_float(r[j]);
                if (p.act_silu == 3) {
                  const uint32_t uword = uw[j >> 1];
                  const float u = __uint_as_float((j & 1) ? (uword & 0xffff0000u) : (uword << 16));
                  r[j] = __float_as_uint(dy * u * dsilu);
                  up_grad[j] = dy * (g * sgm);
                } else {
                  r[j] = __float_as_uint(dy * dsilu);
                }
              }
              if (p.act_silu == 3) {
#pragma unroll
                for (int j = 0; j < 16; ++j) packed_up[h * 16 + j] = pack_bf16x2(up_grad[2 * j], up_grad[2 * j + 1]);
              }
            }
            if constexpr (kEpi == kEpiBf16Grouped) {
              if (keep_before) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  before[h * 16 + j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
              }
            }
            if constexpr (kEpi == kEpiCeBackward) {
              // scale * exp(logit - lse) = exp2(logit*log2e + (log2(scale) - lse*log2e)): one
              // FMA and one ex2 per element; the target and the padding mask are
              // handled only in the 32-column chunk they fall into.
              const int cbase = col0 + c * 64 + h * 32;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                r[j] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(r[j]), kLog2e, neg_lse2)));
              if (p.ce_scale < 0.f) {               // uniform: a negative upstream gradient
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] ^= 0x80000000u;
              }
              const unsigned target_off = static_cast<unsigned>(target - cbase);
              if (target_off < 32u) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (static_cast<unsigned>(j) == target_off) r[j] = __float_as_uint(__uint_as_float(r[j]) - p.ce_scale);
              }
              if (cbase + 32 > p.ce_classes) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (cbase + j >= p.ce_classes) r[j] = 0u;
              }
            }
            if constexpr (kEpi == kEpiBf16Grouped) {
              if (p.act_silu) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  // x * sigmoid(x) = hx + hx * tanh(hx), hx = x / 2: one MUFU op per element
                  const float hx = 0.5f * __uint_as_float(r[j]);
                  r[j] = __float_as_uint(fmaf(hx, fast_tanh(hx), hx));
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j)
              packed[h * 16 + j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
          }
          if (c == kChunks - 1) release_accumulator();
          if constexpr (kEpi == kEpiBf16GroupedActBwd) {
            // SwiGLU: C is the [rows, 2, n] panel, so columns at or beyond n are NOT outside the
            // tensor map (they are the "up" half): a chunk past the product's n columns must not be
            // stored at all, and the gradient of the "up" half goes n columns further on (the host
            // requires n % 64 == 0, so a chunk of gate columns never reaches into it).
            if (col0 + c * 64 < p.n) {
              put_chunk(&p.map_c, p.c_bf16, p.ldc, col0 + c * 64, p.n, packed);
              if (p.act_silu == 3) put_chunk(&p.map_c, p.c_bf16, p.ldc, p.n + col0 + c * 64, 2 * p.n, packed_up);
            }
          } else {
            put_chunk(&p.map_c, p.c_bf16, p.ldc, col0 + c * 64, p.n, packed);
          }
          if constexpr (kEpi == kEpiBf16Grouped) {
            if (keep_before) put_chunk(&p.map_d, p.d_bf16, p.ldd, col0 + c * 64, p.n, before);
          }
          }
        }
      } else if constexpr (kEpi == kEpiCeForward) {
        // Online softmax over this tile's 256 columns of the thread's row.
        constexpr int kChunks = kTileN / 32;
        const int row = row0 + lane;
        if (t.first) {
          run_max = -INFINITY;
          run_sum = 0.f;
          have_target = false;
        }
        const int target = row < p.m ? p.targets[row] : -1;
#pragma unroll 1
        for (int c = 0; c < kChunks; ++c) {
          const int cbase = col0 + c * 32;
          if (cbase >= p.ce_classes) {            // whole chunk is padding (warp-uniform)
            if (c == kChunks - 1) release_accumulator();
            continue;
          }
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c * 32, r);
          tmem_ld_wait();
          if (c == kChunks - 1) release_accumulator();
          // Padding can only start inside the last real chunk; everywhere else the
          // mask is skipped.  The target column is looked for only in its own chunk.
          if (cbase + 32 > p.ce_classes) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (cbase + j >= p.ce_classes) r[j] = __float_as_uint(-INFINITY);
          }
          const unsigned target_off = static_cast<unsigned>(target - cbase);
          if (target_off < 32u) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (static_cast<unsigned>(j) == target_off) target_logit = __uint_as_float(r[j]);
            have_target = true;
          }
          // Four independent chains each for the max and for the sum: one warp per
          // scheduler has no other warp to hide a 32-long dependent chain behind.
          float mx[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) mx[q] = __uint_as_float(r[q]);
#pragma unroll
          for (int j = 4; j < 32; ++j) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(r[j]));
          const float cmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
          const float new_max = fmaxf(run_max, cmax);
          const float m2 = new_max * kLog2e;
          float sm[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int j = 0; j < 32; ++j) sm[j & 3] += fast_exp2(fmaf(__uint_as_float(r[j]), kLog2e, -m2));
          run_sum = run_sum * fast_exp2((run_max - new_max) * kLog2e) + ((sm[0] + sm[1]) + (sm[2] + sm[3]));
          run_max = new_max;
        }
        if (t.last && row < p.m) {
          const int chunk = walk.item / p.tiles_m;
          p.ce_partials[static_cast<long long>(chunk) * p.m + row] = make_float2(run_max, run_sum);
          if (have_target) p.ce_target_logit[row] = target_logit;
        }
      } else {
        // kEpiBf16Rmw: bf16 read-modify-write, thread = row, 32 columns (64 bytes) at a time.
        constexpr int kChunks = kTileN / 32;
        const int row = row0 + lane;
        uint16_t* crow = p.c_bf16 + static_cast<long long>(t.batch) * p.batch_stride_c +
                         static_cast<long long>(row) * p.ldc;
#pragma unroll 1
        for (int c = 0; c < kChunks; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c * 32, r);
          tmem_ld_wait();
          if (c == kChunks - 1) release_accumulator();
          const int col = col0 + c * 32;
          if (row < p.m) {
            if (col + 32 <= p.n) {
              uint4* ptr = reinterpret_cast<uint4*>(crow + col);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 old = ptr[q];
                const uint32_t o[4] = {old.x, old.y, old.z, old.w};
                uint32_t nw[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float lo = __uint_as_float(o[j] << 16) + __uint_as_float(r[q * 8 + 2 * j]);
                  const float hi = __uint_as_float(o[j] & 0xffff0000u) + __uint_as_float(r[q * 8 + 2 * j + 1]);
                  nw[j] = pack_bf16x2(lo, hi);
                }
                ptr[q] = make_uint4(nw[0], nw[1], nw[2], nw[3]);
              }
            } else {
              for (int j = 0; j < 32 && col + j < p.n; ++j) {
                const float v = __uint_as_float(static_cast<uint32_t>(crow[col + j]) << 16) + __uint_as_float(r[j]);
                crow[col + j] = static_cast<uint16_t>(pack_bf16x2(v, 0.f) & 0xffffu);
              }
            }
          }
        }
      }
    }
    if (lane == 0) tma_wait_group<0>();   // all TMA stores of this warp landed before exit
    __syncwarp();
  }

  // ------------------------------------------------------------ teardown
  if (*abort_flag) {
    // Something timed out: give copies that are still in flight time to land
    // before the shared memory they target is released.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tcgen05_fence_before_sync();
  if constexpr (kCtaGroup == 2) cluster_sync(); else __syncthreads();
  tcgen05_fence_after_sync();
  if (warp == 2) tmem_dealloc<kCtaGroup>(tmem_base, kTmemCols);
}

}  // namespace b200
