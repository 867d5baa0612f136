// Flash attention for prompt portions on the 5th-generation tensor cores (sm_100a), over the
// paged bfloat16 cache: Q.K^T and P.V are tcgen05.mma instructions with their accumulators in
// tensor memory; Q, K and V tiles arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle), the
// keys and values page by page through the request's block table.  Formula and masking are the
// reference's (runtime/src/text_model.cpp:83-114); its CUDA kernel handles one query at a time on
// the CUDA cores (cuda/src/cuda_backend.cu:347-395).
//
// A work item = two neighbouring tiles of 128 query rows of one head, A and B (B is missing where a
// segment ends after A), walking the 128-key tiles that they see.  One CTA per SM takes items in turn
// (longest first; see Walk) and runs them through one pipeline that is set up once.  In launches
// with so few tiles that pairs would leave SMs without work (PAIRED = false) an item is one tile:
// tile B's warps then idle and the tile's S takes both S buffers in turn, so that the S of the next
// keys is computed while the softmax of these runs.
//   warps 0, 3    TMA: warp 0 the K tiles, warp 3 the V tiles, into rings of two stages each (three of keys
//                 without pairs) that run on across items.  A tile is eight loads of 16 keys (a page may hold
//                 no more) per 64 dims; lane b looks up block b's page, an elected lane issues all of them.
//                 A key stage is free again as soon as the last Q.K^T that uses it is done, its values'
//                 stage after the last P.V.
//   warp 1        MMA (the whole warp walks the loop and waits, an elected lane issues): for each query tile
//                 in turn, O += P V of the tile's current keys (P read from
//                 tensor memory, V as an MN-major operand from shared memory) as soon as its softmax
//                 warpgroup has written P, then S = Q K^T of the next keys into the tile's S.
//   warp 2        TMA: an item's Q tiles, each as soon as the last Q.K^T of the item before has read
//                 the old one.
//   warps 4..11   softmax of tile A, warps 12..19 of tile B, two warpgroups each.  A query row is
//                 shared by two threads (one per warpgroup, same lane of tensor memory), each owning 64
//                 of the tile's 128 keys: it reads its part of the row of S (once for the maximum, on
//                 which it agrees with its partner through shared memory, and once more, 32 columns
//                 at a time, for the exponentials: few registers a thread), writes the exponentials as
//                 bfloat16 over the first half of its own columns of S (P lives where S was) and keeps
//                 its part of the row sum.  While the warps of one tile wait for their next S (the
//                 tile's P.V and next Q.K^T run then), those of the other compute: every scheduler
//                 of the SM has four softmax warps in two phases to issue from, which keeps the
//                 special-function unit busy (one or two warps a scheduler leave it idle half the time).
// Order in tensor memory: the next Q.K^T into an S buffer overwrites the P in it, so the MMA thread
// issues it only after the P.V that reads that P has finished; with pairs a full S therefore also says
// that the tile's output rows are at rest.  No thread is ever two phases behind a barrier (a parity
// wait cannot tell that from "done"): the P.V completions have a barrier per S buffer for that reason.
// The output rows live in tensor memory and the P.V products accumulate into them; a row's reference
// maximum moves only when the true maximum has grown by more than 2^RESCALE_STEP (then the row in
// tensor memory is scaled down once), so P may reach 2^RESCALE_STEP and most tiles need no work on O.
// Softmax statistics, rescaling and the output sum are float32.  Every mbarrier wait is bounded
// and reports through *err instead of hanging.
#include "tc_common.cuh"

#define K_ST_PAIRS 2        // stages of keys in shared memory with two query tiles an item ...
#define K_ST_SINGLE 3       // ... and with one (the second tile's room holds a stage more)
#define V_ST 2              // stages of values
#define RESCALE_STEP 8.0f
#define QT 128              // query rows per tile
#define KT 128              // keys per tile
#define ATTN_THREADS 640    // warps 0..3: TMA of keys, MMA, TMA of queries, TMA of values; 4..11 and 12..19: softmax

namespace {


struct AttnArgs {
  bf16* out;
  const int* seg_q_start;
  const int* seg_pos0;
  const int* block_table;
  int* err;
  int ld_out, max_blocks, H, Hkv, page, window;
  int segments, q_pairs, items;                      // items = H x segments x q_pairs (some of them empty)
  int paired;                                        // 1: an item is two query tiles; 0: one (q_pairs then counts tiles)
  float scale_log2;
};

// bar.sync over the `count` threads that name barrier `id`
__device__ __forceinline__ void named_barrier(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

struct Item {
  const int* bt;                                     // the segment's row of the block table
  int h, kvh, q0, qlen, tile0, pos0;                 // tile0: first row of tile A in its segment (B: tile0 + 128)
  int k_last, tile_begin;                            // the last key any row of the item sees; its first key tile
  int n_a, n_b;                                      // key tiles of A and of B (0: no B; else n_a or n_a + 1)
};

// Item `idx` of the launch: heads fastest (the heads of one kv head are neighbours and read the same
// keys and values), then segments, then pairs of query tiles from the last pair (which sees the most
// keys) down.  False for a pair beyond its segment's end.
template <bool PAIRED>
__device__ __forceinline__ bool item_at(const AttnArgs& a, int idx, Item& t) {
  t.h = idx % a.H;
  const int rest = idx / a.H;
  const int seg = rest % a.segments, y = rest / a.segments;
  t.q0 = a.seg_q_start[seg];
  t.qlen = a.seg_q_start[seg + 1] - t.q0;
  t.tile0 = (a.q_pairs - 1 - y) * (PAIRED ? 2 * QT : QT);
  if (t.tile0 >= t.qlen) return false;
  t.pos0 = a.seg_pos0[seg];
  t.kvh = t.h / (a.H / a.Hkv);
  t.bt = a.block_table + (size_t)seg * a.max_blocks;
  const int rows = t.qlen - t.tile0;                 // of both tiles
  const int last_a = t.pos0 + t.tile0 + (rows < QT ? rows : QT) - 1;
  int k_first = 0;
  if (a.window > 0) { const int f = t.pos0 + t.tile0 - a.window + 1; k_first = f > 0 ? f : 0; }
  t.tile_begin = k_first / KT;
  t.n_a = last_a / KT - t.tile_begin + 1;
  t.n_b = 0;
  t.k_last = last_a;
  if (PAIRED && rows > QT) {
    t.k_last = t.pos0 + t.tile0 + (rows < 2 * QT ? rows : 2 * QT) - 1;
    t.n_b = t.k_last / KT - t.tile_begin + 1;
  }
  return true;
}

// The items of one CTA: in the order of item_at the items are dealt out in rounds of gridDim.x, to
// and fro (CTA c gets item c of an even round and item gridDim.x - 1 - c of an odd one), so that a
// CTA that got a long item in one round gets a short one in the next.  Every role of the CTA walks
// the same list on its own.
template <bool PAIRED>
struct Walk {
  int round, cta, ctas;
  __device__ bool next(const AttnArgs& a, Item& t) {
    for (;;) {
      const long long first = (long long)round * ctas;
      if (first >= a.items) return false;
      const long long idx = first + ((round & 1) ? ctas - 1 - cta : cta);
      ++round;
      if (idx < a.items && item_at<PAIRED>(a, (int)idx, t)) return true;
    }
  }
};

template <int HD, bool PAIRED>
__global__ void __launch_bounds__(ATTN_THREADS) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                       const __grid_constant__ CUtensorMap map_kv, const AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int NH = HD / 64;                        // 64-element halves of the head
  constexpr int Q_BYTES = QT * HD * 2;               // [NH][128 rows][64]
  constexpr int K_BYTES = KT * HD * 2;               // [NH][128 keys][64]
  constexpr int HALF_BYTES = 128 * 128;              // one [128][64] bf16 tile
  static_assert(2 * KT + 2 * HD <= 512, "S and O of both query tiles must fit tensor memory");
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = base;                                // tiles A and B
  constexpr int K_ST = PAIRED ? K_ST_PAIRS : K_ST_SINGLE;
  uint8_t* sK = sQ + (PAIRED ? 2 : 1) * Q_BYTES;     // K_ST stages
  uint8_t* sV = sK + K_ST * K_BYTES;                 // V_ST stages
  uint64_t* bars = (uint64_t*)(sV + V_ST * K_BYTES);
  uint64_t* q_full = bars;                           // [2]: one per query tile, like the next four
  uint64_t* q_empty = bars + 2;
  uint64_t* s_full = bars + 4;
  uint64_t* p_full = bars + 6;
  uint64_t* pv_done = bars + 8;
  uint64_t* k_full = bars + 10;                      // K_ST each
  uint64_t* k_empty = k_full + K_ST;
  uint64_t* v_full = k_empty + K_ST;                 // V_ST each
  uint64_t* v_empty = v_full + V_ST;
  uint32_t* tmem_slot = (uint32_t*)(v_empty + V_ST);
  // What the two threads of a row tell each other, 256 bytes for each (query tile, quarter of the rows)
  // (the warps of a quarter meet at a barrier of their own): the tile's maxima (bfloat16, rounded up,
  // two tiles in flight: [2][2][32 rows]) and at the end of an item the row sums (float32 [2][32 rows],
  // over the same bytes)
  uint8_t* xchg = (uint8_t*)(bars + 32);

  // the warp's number through a shuffle: the compiler then knows that it is the same in all lanes, and keeps what
  // depends on it alone (the MMA warp's descriptors and counters) in uniform registers
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  pdl_wait();
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int x = 0; x < 2; ++x) {
      mbar_init(&q_full[x], 1); mbar_init(&q_empty[x], 1);
      mbar_init(&s_full[x], 1); mbar_init(&p_full[x], 256); mbar_init(&pv_done[x], 1);
    }
    for (int i = 0; i < K_ST; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < V_ST; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;                  // columns 0..255: S of A and of B (P over the first half of each)
  const uint32_t tmem_o = tmem + 2 * KT;             // 2 x HD columns: the output rows of A and of B

  Walk<PAIRED> walk{0, (int)blockIdx.x, (int)gridDim.x};
  Item t;

  if (warp == 0 || warp == 3) {
    // Warp 0 requests the keys, warp 3 the values, each at the pace of its own ring (in one warp the keys
    // waited for a free stage of values, which comes later than a free stage of keys, and the next Q.K^T
    // found them late).  A tile is 8 blocks of 16 keys (a page may hold no more), each in NH halves of 64
    // dims: up to 16 small TMA loads.  The whole warp walks the items; lane b finds block b's rows in the
    // cache, and an elected lane issues all the loads from values the compiler knows to be the same in all
    // lanes (a lane that issues loads of its own pays for moving their operands to uniform registers).
    const int which = warp == 0 ? 0 : 1;             // 0: keys, 1: values
    const bool leader = elect_one();
    uint64_t* full = which ? v_full : k_full;
    uint64_t* empty = which ? v_empty : k_empty;
    const int stages = which ? V_ST : K_ST;
    uint8_t* ring = which ? sV : sK;
    int s = 0;                                       // the ring's stage, and how often it has been round
    uint32_t lap = 0;
    bool alive = true;
    while (alive && walk.next(a, t)) {
      const int last_block = t.k_last & ~15;
      const int n = t.n_b > t.n_a ? t.n_b : t.n_a;
      for (int j = 0; j < n; ++j) {
        int key0 = (t.tile_begin + j) * KT + (lane & 7) * 16;
        if (key0 > last_block) key0 = last_block;              // keys nobody sees: any valid page will do
        const int pg = t.bt[key0 / a.page];                    // fetched before the wait: its latency is the wait's
        const int my_row = ((pg * 2 + which) * a.Hkv + t.kvh) * a.page + (key0 % a.page);
        alive = mbar_wait(&empty[s], (lap & 1) ^ 1, a.err, 11);
        if (!alive) break;
        if (leader) mbar_expect_tx(&full[s], K_BYTES);
#pragma unroll
        for (int blk = 0; blk < KT / 16; ++blk) {
          const int row = __shfl_sync(0xffffffffu, my_row, blk);
          if (leader) {
#pragma unroll
            for (int hf = 0; hf < NH; ++hf)
              tma_load_2d(ring + s * K_BYTES + hf * HALF_BYTES + blk * 16 * 128, &map_kv, &full[s], hf * 64, row);
          }
        }
        __syncwarp();
        if (++s == stages) { s = 0; ++lap; }
      }
    }
  } else if (warp == 2) {
    {
      const bool leader = elect_one();
      int loads[2] = {0, 0};                         // of tile A and of tile B so far: their barriers' phases
      bool alive = true;
      while (alive && walk.next(a, t)) {
        for (int x = 0; x < 2 && alive; ++x) {
          if (x == 1 && t.n_b == 0) break;
          // the last Q.K^T of the tile loaded before has read the old Q
          alive = mbar_wait(&q_empty[x], (loads[x] & 1) ^ 1, a.err, 10);
          if (!alive) break;
          if (leader) {
            mbar_expect_tx(&q_full[x], Q_BYTES);
            for (int f = 0; f < NH; ++f)
              tma_load_2d(sQ + x * Q_BYTES + f * HALF_BYTES, &map_q, &q_full[x], t.h * HD + f * 64, t.q0 + t.tile0 + x * QT);
          }
          __syncwarp();
          ++loads[x];
        }
      }
    }
  } else if (warp == 1) {
    {
      // The whole warp walks the items and waits; one elected lane issues the products.  (A branch on the lane
      // number around all of this makes every operand of every product a per-thread value, to be moved to the
      // uniform registers the instruction wants, one at a time: some 85 clocks a product.)
      const bool leader = elect_one();
      constexpr uint32_t idesc_qk = umma_idesc(QT, KT, 0);
      constexpr uint32_t idesc_pv = umma_idesc(QT, HD, 1);
      int loads[2] = {0, 0};                         // Q tiles of A and of B seen so far
      int n_pv[2] = {0, 0};                          // P.V products of A and of B issued so far (Q.K^T run one ahead)
      int kbase = 0;                                 // key tiles of all items before this one: the rings' positions
      // S of query tile qx over the item's key tile j, into S buffer x (`last`: no later product reads this Q)
      auto qk = [&](int x, int qx, int j, bool last) -> bool {
        const int g = kbase + j, ks = g % K_ST;
        if (!mbar_wait(&k_full[ks], (g / K_ST) & 1, a.err, 13)) return false;
        // the buffer's last P lies where this S goes: the product that reads it must have finished
        if (n_pv[x] > 0 && !mbar_wait(&pv_done[x], (n_pv[x] - 1) & 1, a.err, 14)) return false;
        tc_fence_after();
        const uint32_t d = tmem + (uint32_t)(x * KT);
        if (leader) {
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) {
          const uint64_t dq = umma_desc(smem_u32(sQ + qx * Q_BYTES + hf * HALF_BYTES));
          const uint64_t dk = umma_desc(smem_u32(sK + ks * K_BYTES + hf * HALF_BYTES));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_f16(d, dq + 2 * kk, dk + 2 * kk, idesc_qk, (hf > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&s_full[x]);
        if (qx == 1 || t.n_b == 0) umma_commit(&k_empty[ks]);  // B (where there is one) is the last to read a key tile
        if (last) umma_commit(&q_empty[qx]);
        }
        __syncwarp();
        return true;
      };
      // O of query tile qx += P V over the item's key tile j, P from S buffer x
      auto pv = [&](int x, int qx, int j) -> bool {
        const int g = kbase + j, vs = g % V_ST;
        if (!mbar_wait(&v_full[vs], (g / V_ST) & 1, a.err, 16)) return false;
        if (!mbar_wait(&p_full[x], n_pv[x] & 1, a.err, 15)) return false;
        tc_fence_after();
        // P [128 rows][128 keys] in tensor memory, two keys per column, each softmax warpgroup's 64 keys at the
        // start of its share of S; V [128 keys][HD] MN-major
        const uint32_t o = tmem_o + (uint32_t)(qx * HD), p = tmem + (uint32_t)(x * KT);
        if (leader) {
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
          const uint32_t v_addr = smem_u32(sV + vs * K_BYTES + (kk * 16) * 128);
          const uint32_t p_col = (uint32_t)(((kk * 16) / 64) * 64 + ((kk * 16) % 64) / 2);
          umma_f16_ts(o, p + p_col, umma_desc_mn(v_addr, HALF_BYTES), idesc_pv, (kk > 0 || j > 0) ? 1u : 0u);
        }
        umma_commit(&pv_done[x]);
        if (qx == 1 || t.n_b == 0) umma_commit(&v_empty[vs]);
        }
        __syncwarp();
        ++n_pv[x];
        return true;
      };
      bool ok = true;
      while (ok && walk.next(a, t)) {
        ok = mbar_wait(&q_full[0], loads[0] & 1, a.err, 12);
        ++loads[0];
        if (!PAIRED) {
          // One query tile an item: its S takes the two S buffers in turn (by the running count of key
          // tiles), so that S of the next keys is computed while the softmax of these runs.
          if (ok) ok = qk(kbase & 1, 0, 0, t.n_a == 1);
          for (int j = 0; j < t.n_a && ok; ++j) {
            if (j + 1 < t.n_a) ok = qk((kbase + j + 1) & 1, 0, j + 1, j + 2 == t.n_a);
            if (ok) ok = pv((kbase + j) & 1, 0, j);
          }
          kbase += t.n_a;
          continue;
        }
        if (ok) ok = qk(0, 0, 0, t.n_a == 1);
        if (ok && t.n_b > 0) {
          ok = mbar_wait(&q_full[1], loads[1] & 1, a.err, 12);
          ++loads[1];
          if (ok) ok = qk(1, 1, 0, t.n_b == 1);
        }
        const int n = t.n_b > t.n_a ? t.n_b : t.n_a;
        for (int j = 0; j < n && ok; ++j) {
          if (j < t.n_a) {
            ok = pv(0, 0, j);
            if (ok && j + 1 < t.n_a) ok = qk(0, 0, j + 1, j + 2 == t.n_a);
          }
          if (ok && j < t.n_b) {
            ok = pv(1, 1, j);
            if (ok && j + 1 < t.n_b) ok = qk(1, 1, j + 1, j + 2 == t.n_b);
          }
        }
        kbase += n;
      }
    }
  } else if (warp >= 4) {
    // softmax: thread = (query row of tile x, half of the tile's keys)
    constexpr int KPT = KT / 2;                        // keys of a tile per thread
    constexpr int OPT = HD / 2;                        // output columns per thread
    const int x = (warp - 4) >> 3;
    const int wg = ((warp - 4) >> 2) & 1;              // which half of the keys and of the output columns
    const int qd = warp & 3;                           // the quarter of tensor memory's lanes this warp may touch
    const int r = qd * 32 + lane;
    const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
    const uint32_t o_addr = tmem_o + lane_base + (uint32_t)(x * HD + wg * OPT);
    bf16* mx_x = (bf16*)(xchg + (x * 4 + qd) * 256);
    float* l_x = (float*)(xchg + (x * 4 + qd) * 256);
    const int bar_id = 1 + x * 4 + qd;
    int n_t = 0;                                       // this tile's key tiles so far: its barriers' phases
    bool ok = true;
    // A wait that gives up makes the whole warp skip the rest of its work, but not the meetings with
    // its partner warp: those are kept to the end, so that nobody waits at a barrier for ever.
    while (walk.next(a, t)) {
      const int n = x ? t.n_b : t.n_a;               // without pairs tile B's warps have nothing to do
      if (n == 0) continue;
      const int row_in_seg = t.tile0 + x * QT + r;
      const int hi = row_in_seg < t.qlen ? t.pos0 + row_in_seg : -1;
      const int lo = (a.window > 0 && hi - a.window + 1 > 0) ? hi - a.window + 1 : 0;
      float m_ref = -INFINITY, l = 0.f;
      for (int j = 0; j < n; ++j, ++n_t) {
        const int key_base = (t.tile_begin + j) * KT + wg * KPT;
        const bool all_visible = key_base >= lo && key_base + KPT - 1 <= hi;   // no mask needed in this part
        // with pairs this tile has S buffer x to itself; a tile alone takes the two buffers in turn
        const int buf = PAIRED ? x : (n_t & 1);
        const uint32_t phase = PAIRED ? (uint32_t)(n_t & 1) : (uint32_t)((n_t >> 1) & 1);
        const uint32_t s_addr = tmem + lane_base + (uint32_t)(buf * KT + wg * KPT);
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&s_full[buf], phase, a.err, 17));
        // first pass over this thread's part of the row of S: its maximum
        float mx = -INFINITY;
        if (ok) {
          tc_fence_after();
          uint32_t sv[KPT];
          tmem_ld32(s_addr, sv);
          tmem_ld32(s_addr + 32, sv + 32);
          tmem_wait_ld();
          if (all_visible) {
            // four independent chains: one chain of dependent maxima would cost more than the loads did
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < KPT; i += 4) {
#pragma unroll
              for (int u = 0; u < 4; ++u) m4[u] = fmaxf(m4[u], __uint_as_float(sv[i + u]));
            }
            mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
          } else {
#pragma unroll
            for (int i = 0; i < KPT; ++i) {
              const int key = key_base + i;
              if (key >= lo && key <= hi) mx = fmaxf(mx, __uint_as_float(sv[i]));
            }
          }
          mx *= a.scale_log2;                            // the scale is positive: max commutes with it
        }
        {
          // The two threads of a row agree on one value: each rounds its maximum up to bfloat16, leaves
          // it for the other and takes the larger.  (The reference maximum need not be the exact one:
          // any common value at or above the true maximum less 2^RESCALE_STEP serves.)
          const bf16 mine = __float2bfloat16_ru(mx);
          bf16* slot = mx_x + (n_t & 1) * 64;
          slot[wg * 32 + lane] = mine;
          named_barrier(bar_id, 64);
          mx = fmaxf(__bfloat162float(mine), __bfloat162float(slot[(wg ^ 1) * 32 + lane]));
        }
        if (!ok) continue;
        float corr = 1.f;
        if (mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY)) {
          corr = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - mx);
          m_ref = mx;
        }
        l *= corr;
        if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
          // Some row of this warp moves its reference: scale this thread's columns of the warp's rows
          // of O (by 1 where nothing moved); the partner warp decides alike, from the same values.
          // With pairs the product of the tile before has finished (this S was issued after it); a
          // tile alone, whose S is computed ahead, waits for it.
          if (!PAIRED) {
            ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(n_t - 1) & 1], (uint32_t)(((n_t - 1) >> 1) & 1), a.err, 18));
            if (!ok) continue;
            tc_fence_after();
          }
#pragma unroll 1
          for (int c = 0; c < OPT; c += 32) {
            uint32_t v[32];
            tmem_ld32(o_addr + c, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
            tmem_st32(o_addr + c, v);
          }
        }
        // second pass, 32 columns at a time:
        // the exponentials, as P over the first half of this thread's columns (a store overwrites
        // only columns that have been read), and their sum
        const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < KPT; c += 32) {
          uint32_t sv[32], w[16];
          tmem_ld32(s_addr + c, sv);
          tmem_wait_ld();
          if (all_visible) {                             // most tiles: no mask, two instructions per score
            float s4[4] = {0.f, 0.f, 0.f, 0.f};          // the row sum in four chains, added in a fixed order
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float e0 = fast_exp2(fmaf(__uint_as_float(sv[i]), a.scale_log2, neg_m));
              const float e1 = fast_exp2(fmaf(__uint_as_float(sv[i + 1]), a.scale_log2, neg_m));
              s4[(i >> 1) & 3] += e0 + e1;
              w[i >> 1] = pack2_bf16(e0, e1);
            }
            sum += (s4[0] + s4[1]) + (s4[2] + s4[3]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float e[2];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int key = key_base + c + i + u;
                e[u] = (key >= lo && key <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[i + u]), a.scale_log2, neg_m)) : 0.f;
              }
              sum += e[0] + e[1];
              w[i >> 1] = pack2_bf16(e[0], e[1]);
            }
          }
          tmem_st16(s_addr + (uint32_t)(c >> 1), w);
        }
        l += sum;
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_full[buf]);
      }
      {
        // the row's sum: both threads' parts, added in the same order by both.  A barrier first (the
        // maxima of the last two tiles lie in the bytes the sums go to) and one after (the next
        // item's maxima go to the same bytes).
        named_barrier(bar_id, 64);
        l_x[wg * 32 + lane] = l;
        named_barrier(bar_id, 64);
        l = l_x[lane] + l_x[32 + lane];
        named_barrier(bar_id, 64);
      }
      if (ok) {
        ok = PAIRED ? __all_sync(0xffffffffu, mbar_wait(&pv_done[x], (uint32_t)((n_t - 1) & 1), a.err, 20))
                      : __all_sync(0xffffffffu, mbar_wait(&pv_done[(n_t - 1) & 1], (uint32_t)(((n_t - 1) >> 1) & 1), a.err, 20));
        tc_fence_after();
        // every lane takes part in the loads (they are warp-wide); only rows of the segment are stored
        const bool store = ok && row_in_seg < t.qlen;
        const float inv = store ? 1.f / l : 0.f;
        bf16* orow = a.out + (size_t)(t.q0 + (store ? row_in_seg : 0)) * a.ld_out + (size_t)t.h * HD + wg * OPT;
#pragma unroll 1
        for (int c = 0; c < OPT; c += 32) {
          uint32_t v[32];
          tmem_ld32(o_addr + c, v);
          tmem_wait_ld();
          if (store) {
#pragma unroll
            for (int i = 0; i < 32; i += 8)
              *(uint4*)(orow + c + i) = make_uint4(pack2_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv),
                                                   pack2_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv),
                                                   pack2_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv),
                                                   pack2_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv));
          }
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

int device_sms() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

template <int HD, bool PAIRED>
int launch(const CUtensorMap& mq, const CUtensorMap& mkv, const AttnArgs& args, cudaStream_t st) {
  // two Q tiles, the rings of keys and values, 256 bytes of barriers, 2 KB for what a row's threads exchange, 1 KB to align
  constexpr int smem = 2 * QT * HD * 2 + (K_ST_PAIRS + V_ST) * KT * HD * 2 + 256 + 2048 + 1024;
  static_assert(QT * HD * 2 + (K_ST_SINGLE + V_ST) * KT * HD * 2 <= 2 * QT * HD * 2 + (K_ST_PAIRS + V_ST) * KT * HD * 2, "one layout's room serves both");
  static_assert(smem <= 227 * 1024, "more shared memory than a CTA can have");
  static bool configured = false;
  auto kernel = attn_prefill_tc_kernel<HD, PAIRED>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  // one CTA per SM, or one per item when there are fewer
  const int ctas = args.items < device_sms() ? args.items : device_sms();
  return qv_launch(kernel, dim3(ctas), dim3(ATTN_THREADS), (size_t)smem, st, mq, mkv, args);
}

}  // namespace

// Prompt portions (any mix of segments) at head sizes 64 and 128.  q: [T, ld_q] with the heads of a
// token side by side (row r of the q tensor map); cache: [cache_pages][2][Hkv][page][hd].  Refuses
// (QV_ERR_UNSUPPORTED) other head sizes, pages that are no multiple of 16 and unaligned operands.
extern "C" int qv_attn_prefill_tc(void* out, int ld_out, const void* q, int ld_q, int T, const void* cache, long long cache_pages,
                                  const int* seg_q_start, const int* seg_pos0, const int* block_table, int max_blocks, int S,
                                  int max_q_len, int max_ctx_len, int H, int Hkv, int hd, int page, int window, float scale, int* err,
                                  void* stream) {
  if (S <= 0 || max_q_len <= 0) return 0;
  if ((hd != 64 && hd != 128) || Hkv <= 0 || H % Hkv || page % 16 || (ld_q & 7) || (ld_out & 7) || ((uintptr_t)q & 15) ||
      ((uintptr_t)cache & 15) || ((uintptr_t)out & 15))
    return QV_ERR_UNSUPPORTED;
  // Two query tiles an item where that still gives every SM an item, for prompts from (near) their start, whose
  // items grow from one key tile to many: pairs read keys and values once for two tiles and halve the number
  // of items (2,048 tokens 50.2 against 56.1 us, 4,096 tokens 151 against 167 us; 1,024 tokens, 128 pairs
  // on 148 SMs, 26.5 against 21.3 us).  Portions that lie deep in their requests (max_ctx_len, the longest
  // context among them, at least twice the longest portion; 0: not known) have items of equal length, and a
  // launch then costs its rounds of items, a round of pairs about two rounds of single tiles: pairs where
  // they need no more than half the rounds (2,048 tokens ending at 8,192: 4 rounds against 2, 277 against
  // 248 us), single tiles else (1,536 ending at 8,192: 3 rounds against 2, 217 against 246 us).
  const long long sms = device_sms();
  const long long q_tiles = (max_q_len + QT - 1) / QT;
  const long long items_single = (long long)H * S * q_tiles;
  const long long items_paired = (long long)H * S * ((q_tiles + 1) / 2);
  const bool deep = max_ctx_len > 0 && max_ctx_len >= 2 * max_q_len;
  const long long rounds_single = (items_single + sms - 1) / sms, rounds_paired = (items_paired + sms - 1) / sms;
  const int paired = (items_paired >= sms && (!deep || 2 * rounds_paired <= rounds_single)) ? 1 : 0;
  const long long q_pairs = paired ? (q_tiles + 1) / 2 : q_tiles;
  if ((long long)H * S * q_pairs > (1LL << 30)) return QV_ERR_TOO_LARGE;
  CUtensorMap mq, mkv;
  if (!make_map(&mq, q, T, H * hd, ld_q, QT)) return QV_ERR_UNSUPPORTED;
  if (!make_map(&mkv, cache, cache_pages * 2 * Hkv * page, hd, hd, 16)) return QV_ERR_UNSUPPORTED;
  AttnArgs a;
  a.out = (bf16*)out; a.seg_q_start = seg_q_start; a.seg_pos0 = seg_pos0; a.block_table = block_table; a.err = err;
  a.ld_out = ld_out; a.max_blocks = max_blocks; a.H = H; a.Hkv = Hkv; a.page = page; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.segments = S; a.q_pairs = (int)q_pairs; a.items = (int)(H * S * q_pairs); a.paired = paired;
  if (hd == 128) return paired ? launch<128, true>(mq, mkv, a, (cudaStream_t)stream) : launch<128, false>(mq, mkv, a, (cudaStream_t)stream);
  return paired ? launch<64, true>(mq, mkv, a, (cudaStream_t)stream) : launch<64, false>(mq, mkv, a, (cudaStream_t)stream);
}
