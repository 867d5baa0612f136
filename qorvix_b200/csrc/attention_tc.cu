// Flash attention for prompt portions on the 5th-generation tensor cores (sm_100a), over the
// paged bfloat16 cache: Q.K^T and P.V are tcgen05.mma instructions with their accumulators in
// tensor memory; Q, K and V tiles arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle), the
// keys and values page by page through the request's block table.  Formula and masking are the
// reference's (runtime/src/text_model.cpp:83-114); its CUDA kernel handles one query at a time on
// the CUDA cores (cuda/src/cuda_backend.cu:347-395).
//
// A work item = 128 query rows of one head, walking 128-key tiles.  One CTA per SM takes items in turn
// (longest first; see Walk) and runs them through one pipeline that never drains between items:
//   warp 0        TMA: an item's Q as soon as the last Q.K^T of the item before has read the old one,
//                 and K and V tiles into rings of three stages each that run on across items, every
//                 lane issuing one of a stage's loads (a page may hold no more than 16 keys).  Keys
//                 and values have barriers of their own: a key stage is free again as soon as its
//                 Q.K^T is done, two products earlier than its values.
//   warp 1        MMA: S[g] = Q K^T into one of two S buffers in tensor memory (so that S[g+1] is
//                 computed while the softmax of tile g runs), then O += P V with P read from
//                 tensor memory and V as an MN-major operand from shared memory.  O has two buffers
//                 too, one per item in turn: the first products of the next item run while the
//                 softmax warps still write the last item's output.
//   warps 2..     softmax, WGS warpgroups of four warps.  A query row is shared by WGS threads (one
//                 per warpgroup, same lane of tensor memory), each owning 128 / WGS of the tile's keys:
//                 it reads its part of the row of S once, agrees with its partners on the row's
//                 reference maximum through shared memory, writes its exponentials as bfloat16 over
//                 the first half of its own columns of S (P lives where S was, which leaves room
//                 for the second O) and keeps its part of the row sum.
// Order in tensor memory: Q.K^T of tile g+2 overwrites the P of tile g, so the MMA thread issues it only
// after P.V of tile g has finished, and that product was issued only after every softmax thread had read
// its S and arrived for tile g.  A softmax warp may run a tile ahead of the others.  The products'
// completions therefore go to two barriers in turn: a warp that waits for the last product while the one
// before is still running would be two phases ahead of a single barrier, and a parity wait cannot tell
// that from "done".
// The output row lives in tensor memory and the P.V products accumulate into it; a row's reference
// maximum moves only when the true maximum has grown by more than 2^RESCALE_STEP (then the row in
// tensor memory is scaled down once, after the product before has finished), so P may reach
// 2^RESCALE_STEP and most tiles need no work on O.
// Softmax statistics, rescaling and the output sum are float32.  Every mbarrier wait is bounded
// and reports through *err instead of hanging.
#include "tc_common.cuh"

#define KV_ST 3             // stages of keys and values in shared memory
#define RESCALE_STEP 8.0f
#define QT 128              // query rows per item
#define KT 128              // keys per tile
#define SOFTMAX_WGS 2       // warpgroups that share the softmax of a tile (1 or 2)

namespace {

struct AttnArgs {
  bf16* out;
  const int* seg_q_start;
  const int* seg_pos0;
  const int* block_table;
  int* err;
  int ld_out, max_blocks, H, Hkv, page, window;
  int segments, q_tiles, items;                      // items = H x segments x q_tiles (some of them empty)
  float scale_log2;
};

// bar.sync over the `count` threads that name barrier `id`
__device__ __forceinline__ void named_barrier(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

struct Item {
  const int* bt;                                     // the segment's row of the block table
  int h, kvh, q0, qlen, tile0, pos0, k_last, tile_begin, n_tiles;
};

// Item `idx` of the launch: heads fastest (the heads of one kv head are neighbours and read the same
// keys and values), then segments, then query tiles from the last one (which sees the most keys)
// down.  False for a tile beyond its segment's end.
__device__ __forceinline__ bool item_at(const AttnArgs& a, int idx, Item& t) {
  t.h = idx % a.H;
  const int rest = idx / a.H;
  const int seg = rest % a.segments, y = rest / a.segments;
  t.q0 = a.seg_q_start[seg];
  t.qlen = a.seg_q_start[seg + 1] - t.q0;
  t.tile0 = (a.q_tiles - 1 - y) * QT;
  if (t.tile0 >= t.qlen) return false;
  t.pos0 = a.seg_pos0[seg];
  t.kvh = t.h / (a.H / a.Hkv);
  t.bt = a.block_table + (size_t)seg * a.max_blocks;
  const int rows_here = t.qlen - t.tile0 < QT ? t.qlen - t.tile0 : QT;
  t.k_last = t.pos0 + t.tile0 + rows_here - 1;
  int k_first = 0;
  if (a.window > 0) { const int f = t.pos0 + t.tile0 - a.window + 1; k_first = f > 0 ? f : 0; }
  t.tile_begin = k_first / KT;
  t.n_tiles = t.k_last / KT - t.tile_begin + 1;
  return true;
}

// The items of one CTA: in the order of item_at the items are dealt out in rounds of gridDim.x, to
// and fro (CTA c gets item c of an even round and item gridDim.x - 1 - c of an odd one), so that a
// CTA that got a long item in one round gets a short one in the next.  Every role of the CTA walks
// the same list on its own.
struct Walk {
  int round, cta, ctas;
  __device__ bool next(const AttnArgs& a, Item& t) {
    for (;;) {
      const long long first = (long long)round * ctas;
      if (first >= a.items) return false;
      const long long idx = first + ((round & 1) ? ctas - 1 - cta : cta);
      ++round;
      if (idx < a.items && item_at(a, (int)idx, t)) return true;
    }
  }
};

template <int HD, int WGS>
__global__ void __launch_bounds__(64 + 128 * WGS) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                         const __grid_constant__ CUtensorMap map_kv, const AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int NH = HD / 64;                        // 64-element halves of the head
  constexpr int Q_BYTES = QT * HD * 2;               // [NH][128 rows][64]
  constexpr int K_BYTES = KT * HD * 2;               // [NH][128 keys][64]
  constexpr int HALF_BYTES = 128 * 128;              // one [128][64] bf16 tile
  constexpr int KPT = KT / WGS;                      // keys of a tile per softmax thread
  constexpr int OPT = HD / WGS;                      // output columns per softmax thread
  static_assert(WGS == 1 || WGS == 2, "one or two softmax warpgroups");
  static_assert(KPT % 64 == 0 && OPT % 32 == 0, "a thread's keys come in chunks of 64, its output columns in chunks of 32");
  static_assert(2 * KT + 2 * HD <= 512, "S and O, two buffers each, must fit tensor memory");
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = base;
  uint8_t* sK = sQ + Q_BYTES;                        // KV_ST stages
  uint8_t* sV = sK + KV_ST * K_BYTES;                // KV_ST stages
  uint64_t* bars = (uint64_t*)(sV + KV_ST * K_BYTES);
  uint64_t* q_full = bars;                           // 1
  uint64_t* q_empty = bars + 1;                      // 1
  uint64_t* s_full = bars + 2;                       // 2
  uint64_t* p_full = bars + 4;                       // 2
  uint64_t* pv_full = bars + 6;                      // 2
  uint64_t* k_full = bars + 8;                       // KV_ST each
  uint64_t* k_empty = k_full + KV_ST;
  uint64_t* v_full = k_empty + KV_ST;
  uint64_t* v_empty = v_full + KV_ST;
  uint32_t* tmem_slot = (uint32_t*)(v_empty + KV_ST);
  // What the threads of a row tell each other, 256 bytes for each quarter of the rows (the warps of
  // a quarter meet at a barrier of their own and run ahead of or behind the other quarters): the
  // tile's maxima (bfloat16, rounded up, two tiles in flight: [2][WGS][32 rows]) and at the end of
  // an item the row sums (float32 [WGS][32 rows], over the same bytes)
  uint8_t* xchg = (uint8_t*)(bars + 32);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < KV_ST; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 128 * WGS); }
    mbar_init(&pv_full[0], 1); mbar_init(&pv_full[1], 1);
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
  const uint32_t tmem = *tmem_slot;                  // columns 0..255: S, two buffers (P over the first half of each thread's share)
  const uint32_t tmem_o = tmem + 2 * KT;             // 2 x HD columns: the output rows, two buffers

  Walk walk{0, (int)blockIdx.x, (int)gridDim.x};
  Item t;
  // `it` counts this CTA's items, `g` its key tiles over all items: rings and buffers are indexed by them

  if (warp == 0) {
    // The whole warp requests: a tile of keys and values is 8 blocks of 16 keys (a page may hold no
    // more), each in NH halves of 64 dims, i.e. up to 32 small TMA loads.  One thread issuing them
    // all took as long as the tile's softmax; the lanes issue one load each.
    const int which = lane / (8 * NH);               // 0: keys, 1: values (lanes beyond have nothing to do)
    const int blk = (lane % (8 * NH)) / NH, hf = lane % NH;
    if (which < 2) {
      // the lanes that load keys and the lanes that load values each follow their own barriers
      const int leader = which * 8 * NH;
      const unsigned group = ((1u << (8 * NH)) - 1u) << leader;
      uint64_t* full = which ? v_full : k_full;
      uint64_t* empty = which ? v_empty : k_empty;
      uint8_t* dst = (which ? sV : sK) + hf * HALF_BYTES + blk * 16 * 128;
      int g = 0;
      bool alive = true;
      for (int it = 0; alive && walk.next(a, t); ++it) {
        if (lane == 0) {
          // the last Q.K^T of the item before has read the old Q
          alive = mbar_wait(q_empty, (it & 1) ^ 1, a.err, 10);
          if (alive) {
            mbar_expect_tx(q_full, Q_BYTES);
            for (int f = 0; f < NH; ++f) tma_load_2d(sQ + f * HALF_BYTES, &map_q, q_full, t.h * HD + f * 64, t.q0 + t.tile0);
          }
        }
        const int last_block = t.k_last & ~15;
        for (int j = 0; j < t.n_tiles; ++j, ++g) {
          const int s = g % KV_ST;
          int key0 = (t.tile_begin + j) * KT + blk * 16;
          if (key0 > last_block) key0 = last_block;            // keys nobody sees: any valid page will do
          const int pg = t.bt[key0 / a.page];                  // fetched before the wait: its latency is the wait's
          int ok = 1;
          if (lane == leader) {
            ok = alive && mbar_wait(&empty[s], ((g / KV_ST) & 1) ^ 1, a.err, 11) ? 1 : 0;
            if (ok) mbar_expect_tx(&full[s], K_BYTES);
          }
          ok = __shfl_sync(group, ok, leader);
          if (!ok) { alive = false; break; }
          const int row = ((pg * 2 + which) * a.Hkv + t.kvh) * a.page + (key0 % a.page);
          tma_load_2d(dst + s * K_BYTES, &map_kv, &full[s], hf * 64, row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(QT, KT, 0);
      constexpr uint32_t idesc_pv = umma_idesc(QT, HD, 1);
      int pv_issued = 0;                             // P.V products issued so far (= committed to pv_full)
      // S of key tile gt; `last`: no later product of the item reads Q
      auto issue_qk = [&](int gt, bool last) -> bool {
        const int ks = gt % KV_ST;
        if (!mbar_wait(&k_full[ks], (gt / KV_ST) & 1, a.err, 13)) return false;
        // This S goes where the P of two tiles ago lies (and the one after the next where the last P
        // lies): the products that read them must have finished.  Waiting for the last one issued
        // covers both; it was issued a softmax ago, so this costs the softmax warps nothing.
        if (pv_issued > 0 && !mbar_wait(&pv_full[(pv_issued - 1) & 1], ((pv_issued - 1) >> 1) & 1, a.err, 14)) return false;
        tc_fence_after();
        const uint32_t d = tmem + (uint32_t)((gt & 1) * KT);
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) {
          const uint64_t dq = umma_desc(smem_u32(sQ + hf * HALF_BYTES));
          const uint64_t dk = umma_desc(smem_u32(sK + ks * K_BYTES + hf * HALF_BYTES));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_f16(d, dq + 2 * kk, dk + 2 * kk, idesc_qk, (hf > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&s_full[gt & 1]);
        umma_commit(&k_empty[ks]);                   // the keys' stage is free once this product has read it
        if (last) umma_commit(q_empty);
        return true;
      };
      int g = 0;
      bool ok = true;
      for (int it = 0; ok && walk.next(a, t); ++it) {
        ok = mbar_wait(q_full, it & 1, a.err, 12);
        if (ok) ok = issue_qk(g, t.n_tiles == 1);
        const uint32_t o = tmem_o + (uint32_t)((it & 1) * HD);
        for (int j = 0; j < t.n_tiles && ok; ++j, ++g) {
          if (j + 1 < t.n_tiles) ok = issue_qk(g + 1, j + 2 == t.n_tiles);
          if (!ok) break;
          const int s = g % KV_ST;                   // the stage of this tile's values
          if (!mbar_wait(&v_full[s], (g / KV_ST) & 1, a.err, 16)) { ok = false; break; }
          if (!mbar_wait(&p_full[g & 1], (g >> 1) & 1, a.err, 15)) { ok = false; break; }
          tc_fence_after();
          // P [128 rows][128 keys] in tensor memory, two keys per column, each softmax warpgroup's share
          // at the start of its share of S; V [128 keys][HD] MN-major
          const uint32_t p = tmem + (uint32_t)((g & 1) * KT);
#pragma unroll
          for (int kk = 0; kk < KT / 16; ++kk) {
            const uint32_t v_addr = smem_u32(sV + s * K_BYTES + (kk * 16) * 128);
            const uint32_t p_col = (uint32_t)(((kk * 16) / KPT) * KPT + ((kk * 16) % KPT) / 2);
            umma_f16_ts(o, p + p_col, umma_desc_mn(v_addr, HALF_BYTES), idesc_pv, (kk > 0 || j > 0) ? 1u : 0u);
          }
          umma_commit(&pv_full[g & 1]);
          umma_commit(&v_empty[s]);
          ++pv_issued;
        }
      }
    }
  } else {
    // softmax: thread = (query row, share of the tile's keys)
    const int qd = warp & 3;                           // the quarter of tensor memory's lanes this warp may touch
    const int wg = (warp - 2) >> 2;                    // which share of the keys and of the output columns
    const int r = qd * 32 + lane;
    const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
    bf16* mx_x = (bf16*)(xchg + qd * 256);
    float* l_x = (float*)(xchg + qd * 256);
    int g = 0;
    bool ok = true;
    // A wait that gives up makes the whole warp skip the rest of its work, but not the meetings with
    // its partner warps: those are kept to the end, so that nobody waits at a barrier for ever.
    for (int it = 0; walk.next(a, t); ++it) {
      const int row_in_seg = t.tile0 + r;
      const int hi = row_in_seg < t.qlen ? t.pos0 + row_in_seg : -1;
      const int lo = (a.window > 0 && hi - a.window + 1 > 0) ? hi - a.window + 1 : 0;
      const uint32_t o_addr = tmem_o + lane_base + (uint32_t)((it & 1) * HD + wg * OPT);
      float m_ref = -INFINITY, l = 0.f;
      for (int j = 0; j < t.n_tiles; ++j, ++g) {
        const int s = g & 1;
        const int key_base = (t.tile_begin + j) * KT + wg * KPT;
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&s_full[s], (g >> 1) & 1, a.err, 17));
        float mx = -INFINITY;
        uint32_t sv[KPT];                                  // this thread's part of the row of S, read once
        const bool all_visible = key_base >= lo && key_base + KPT - 1 <= hi;   // no mask needed in this part
        const uint32_t s_addr = tmem + lane_base + (uint32_t)(s * KT + wg * KPT);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < KPT; c += 32) tmem_ld32(s_addr + c, sv + c);
          tmem_wait_ld();
          if (all_visible) {
            // four independent chains: one chain of KPT dependent maxima would cost more than the loads did
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
        if (WGS > 1) {
          // The threads of a row agree on one value: each rounds its maximum up to bfloat16, leaves it
          // for the others and takes the largest.  (The reference maximum need not be the exact one:
          // any common value at or above the true maximum less 2^RESCALE_STEP serves.)
          const bf16 mine = __float2bfloat16_ru(mx);
          bf16* slot = mx_x + (g & 1) * (WGS * 32);
          slot[wg * 32 + lane] = mine;
          named_barrier(1 + qd, 32 * WGS);
          mx = __bfloat162float(mine);
#pragma unroll
          for (int w = 0; w < WGS; ++w) mx = fmaxf(mx, __bfloat162float(slot[w * 32 + lane]));
        }
        if (!ok) continue;
        float corr = 1.f;
        if (mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY)) {
          corr = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - mx);
          m_ref = mx;
        }
        l *= corr;
        float sum = 0.f;
        const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
        uint32_t w[KPT / 2];
#pragma unroll
        for (int c = 0; c < KPT; c += 64) {
          if (all_visible) {                             // most tiles: no mask, two instructions per score
            float s4[4] = {0.f, 0.f, 0.f, 0.f};          // the row sum in four chains, added in a fixed order
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
              const float e0 = fast_exp2(fmaf(__uint_as_float(sv[c + i]), a.scale_log2, neg_m));
              const float e1 = fast_exp2(fmaf(__uint_as_float(sv[c + i + 1]), a.scale_log2, neg_m));
              s4[(i >> 1) & 3] += e0 + e1;
              w[(c + i) >> 1] = pack2_bf16(e0, e1);
            }
            sum += (s4[0] + s4[1]) + (s4[2] + s4[3]);
          } else {
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
              float e[2];
#pragma unroll
              for (int x = 0; x < 2; ++x) {
                const int key = key_base + c + i + x;
                e[x] = (key >= lo && key <= hi) ? fast_exp2(fmaf(__uint_as_float(sv[c + i + x]), a.scale_log2, neg_m)) : 0.f;
              }
              sum += e[0] + e[1];
              w[(c + i) >> 1] = pack2_bf16(e[0], e[1]);
            }
          }
        }
        l += sum;
        if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
          // Some row of this warp moves its reference: once the product of the tile before has come
          // to rest, scale this thread's columns of the warp's rows of O (by 1 where nothing moved);
          // the partner warps decide alike, from the same values.
          ok = __all_sync(0xffffffffu, mbar_wait(&pv_full[(g - 1) & 1], ((g - 1) >> 1) & 1, a.err, 18));
          if (!ok) continue;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < OPT; c += 32) {
            uint32_t v[32];
            tmem_ld32(o_addr + c, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
            tmem_st32(o_addr + c, v);
          }
        }
        // P over the first half of this thread's own columns of S (all of which it has read)
#pragma unroll
        for (int c = 0; c < KPT; c += 64) tmem_st32(s_addr + (uint32_t)(c >> 1), w + (c >> 1));
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_full[s]);
      }
      if (WGS > 1) {
        // the row's sum: every thread's part, added in the same order by all of them.  A barrier
        // first (the maxima of the last two tiles lie in the bytes the sums go to) and one after
        // (the next item's maxima go to the same bytes).
        named_barrier(1 + qd, 32 * WGS);
        l_x[wg * 32 + lane] = l;
        named_barrier(1 + qd, 32 * WGS);
        l = 0.f;
#pragma unroll
        for (int w = 0; w < WGS; ++w) l += l_x[w * 32 + lane];
        named_barrier(1 + qd, 32 * WGS);
      }
      if (ok) {
        ok = __all_sync(0xffffffffu, mbar_wait(&pv_full[(g - 1) & 1], ((g - 1) >> 1) & 1, a.err, 20));
        tc_fence_after();
        // every lane takes part in the loads (they are warp-wide); only rows of the segment are stored
        const bool store = ok && row_in_seg < t.qlen;
        const float inv = store ? 1.f / l : 0.f;
        bf16* orow = a.out + (size_t)(t.q0 + (store ? row_in_seg : 0)) * a.ld_out + (size_t)t.h * HD + wg * OPT;
#pragma unroll
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

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mkv, const AttnArgs& args, cudaStream_t st) {
  // Q, the ring of keys and values, 256 bytes of barriers, 1 KB for what a row's threads exchange, 1 KB to align
  constexpr int smem = QT * HD * 2 + 2 * KV_ST * KT * HD * 2 + 256 + 1024 + 1024;
  static_assert(smem <= 227 * 1024, "more shared memory than a CTA can have");
  static bool configured = false;
  auto kernel = attn_prefill_tc_kernel<HD, SOFTMAX_WGS>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  // one CTA per SM, or one per item when there are fewer
  const int ctas = args.items < device_sms() ? args.items : device_sms();
  return qv_launch(kernel, dim3(ctas), dim3(64 + 128 * SOFTMAX_WGS), (size_t)smem, st, mq, mkv, args);
}

}  // namespace

// Prompt portions (any mix of segments) at head sizes 64 and 128.  q: [T, ld_q] with the heads of a
// token side by side (row r of the q tensor map); cache: [cache_pages][2][Hkv][page][hd].  Refuses
// (QV_ERR_UNSUPPORTED) other head sizes, pages that are no multiple of 16 and unaligned operands.
extern "C" int qv_attn_prefill_tc(void* out, int ld_out, const void* q, int ld_q, int T, const void* cache, long long cache_pages,
                                  const int* seg_q_start, const int* seg_pos0, const int* block_table, int max_blocks, int S,
                                  int max_q_len, int H, int Hkv, int hd, int page, int window, float scale, int* err, void* stream) {
  if (S <= 0 || max_q_len <= 0) return 0;
  if ((hd != 64 && hd != 128) || Hkv <= 0 || H % Hkv || page % 16 || (ld_q & 7) || (ld_out & 7) || ((uintptr_t)q & 15) ||
      ((uintptr_t)cache & 15) || ((uintptr_t)out & 15))
    return QV_ERR_UNSUPPORTED;
  const long long q_tiles = (max_q_len + QT - 1) / QT;
  if ((long long)H * S * q_tiles > (1LL << 30)) return QV_ERR_TOO_LARGE;
  CUtensorMap mq, mkv;
  if (!make_map(&mq, q, T, H * hd, ld_q, QT)) return QV_ERR_UNSUPPORTED;
  if (!make_map(&mkv, cache, cache_pages * 2 * Hkv * page, hd, hd, 16)) return QV_ERR_UNSUPPORTED;
  AttnArgs a;
  a.out = (bf16*)out; a.seg_q_start = seg_q_start; a.seg_pos0 = seg_pos0; a.block_table = block_table; a.err = err;
  a.ld_out = ld_out; a.max_blocks = max_blocks; a.H = H; a.Hkv = Hkv; a.page = page; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.segments = S; a.q_tiles = (int)q_tiles; a.items = (int)(H * S * q_tiles);
  if (hd == 128) return launch<128>(mq, mkv, a, (cudaStream_t)stream);
  return launch<64>(mq, mkv, a, (cudaStream_t)stream);
}
