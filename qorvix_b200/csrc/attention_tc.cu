// Flash attention for prompt portions on the 5th-generation tensor cores (sm_100a), over the
// paged bfloat16 cache: Q.K^T and P.V are tcgen05.mma instructions with their accumulators in
// tensor memory; Q, K and V tiles arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle), the
// keys and values page by page through the request's block table.  Formula and masking are the
// reference's (runtime/src/text_model.cpp:83-114); its CUDA kernel handles one query at a time on
// the CUDA cores (cuda/src/cuda_backend.cu:347-395).
//
// One CTA = 128 query rows of one head, walking 128-key tiles:
//   warp 0        TMA: Q once, then K and V tiles into rings of three stages each, every lane issuing
//                 one of a stage's loads (a page may hold no more than 16 keys).  Keys and values
//                 have barriers of their own: a key stage is free again as soon as its Q.K^T is done,
//                 two products earlier than its values, so that the next keys are under way long
//                 before the tensor pipe asks for them.
//   warp 1        MMA: S[j] = Q K_j^T into one of two S buffers in tensor memory (so that S[j+1] is
//                 computed while the softmax of tile j runs), then O += P_j V_j with P read from
//                 tensor memory and V as an MN-major operand from shared memory
//   warps 2..     softmax, WGS warpgroups of four warps.  A query row is shared by WGS threads (one
//                 per warpgroup, same lane of tensor memory), each owning 128 / WGS of the tile's keys:
//                 it reads its part of the row of S once, agrees with its partners on the row's
//                 reference maximum through shared memory, writes its exponentials as bfloat16 into
//                 P's columns in tensor memory and keeps its part of the row sum.  With two
//                 warpgroups every scheduler of the SM has two softmax warps to issue from and each
//                 thread half the exponentials, which is what bounds the one-warpgroup form.
// The output row lives in tensor memory and the P.V products accumulate into it; a row's reference
// maximum moves only when the true maximum has grown by more than 2^RESCALE_STEP (then the row in
// tensor memory is scaled down once), so P may reach 2^RESCALE_STEP and most tiles need no work on O.
// Softmax statistics, rescaling and the output sum are float32.  Every mbarrier wait is bounded
// and reports through *err instead of hanging.
#include "tc_common.cuh"

#define KV_ST 3             // stages of keys and values in shared memory
#define RESCALE_STEP 8.0f
#define QT 128              // query rows per CTA
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
  float scale_log2;
};

// bar.sync over the `count` threads that name barrier `id`
__device__ __forceinline__ void named_barrier(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

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
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = base;
  uint8_t* sK = sQ + Q_BYTES;                        // KV_ST stages
  uint8_t* sV = sK + KV_ST * K_BYTES;                // KV_ST stages
  uint64_t* bars = (uint64_t*)(sV + KV_ST * K_BYTES);
  uint64_t* q_full = bars;                           // 1
  uint64_t* s_full = bars + 1;                       // 2
  uint64_t* s_empty = bars + 3;                      // 2
  uint64_t* p_full = bars + 5;
  uint64_t* p_empty = bars + 6;
  uint64_t* pv_full = bars + 7;
  uint64_t* k_full = bars + 8;                       // KV_ST each
  uint64_t* k_empty = k_full + KV_ST;
  uint64_t* v_full = k_empty + KV_ST;
  uint64_t* v_empty = v_full + KV_ST;
  uint32_t* tmem_slot = (uint32_t*)(v_empty + KV_ST);
  // What the threads of a row tell each other, 256 bytes for each quarter of the rows (the warps of
  // a quarter meet at a barrier of their own and run ahead of or behind the other quarters): the
  // tile's maxima (bfloat16, rounded up, two tiles in flight: [2][WGS][32 rows]) and at the end the
  // row sums (float32 [WGS][32 rows], over the same bytes)
  uint8_t* xchg = (uint8_t*)(bars + 32);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Grid (heads, query tiles, segments): CTAs are handed out in x-fastest order, so all heads of the
  // last query tile (which sees the most keys) start first, then all heads of the tile before, ...:
  // longest work first, which on 148 SMs ends ~30 % earlier than an order that mixes heavy and light
  // CTAs.  The heads of one kv head are neighbours and read the same keys and values.
  const int seg = blockIdx.z, h = blockIdx.x;
  pdl_wait();
  pdl_launch_dependents();
  const int q0 = a.seg_q_start[seg], qlen = a.seg_q_start[seg + 1] - q0;
  const int tile0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * QT;
  if (tile0 >= qlen) return;
  const int pos0 = a.seg_pos0[seg];
  const int kvh = h / (a.H / a.Hkv);
  const int* bt = a.block_table + (size_t)seg * a.max_blocks;
  const int rows_here = qlen - tile0 < QT ? qlen - tile0 : QT;
  const int k_last = pos0 + tile0 + rows_here - 1;
  int k_first = 0;
  if (a.window > 0) { const int f = pos0 + tile0 - a.window + 1; k_first = f > 0 ? f : 0; }
  const int tile_begin = k_first / KT, n_tiles = k_last / KT - tile_begin + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < KV_ST; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 128 * WGS); }
    mbar_init(p_full, 128 * WGS); mbar_init(p_empty, 1); mbar_init(pv_full, 1);
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
  const uint32_t tmem = *tmem_slot;                  // columns 0..255: S, double-buffered
  const uint32_t tmem_pv = tmem + 256;               // HD columns: the output rows
  const uint32_t tmem_p = tmem + 384;                // 64 columns: a row of P, two keys per column

  if (warp == 0) {
    // The whole warp requests: a tile of keys and values is 8 blocks of 16 keys (a page may hold no
    // more), each in NH halves of 64 dims, i.e. up to 32 small TMA loads.  One thread issuing them
    // all took as long as the tile's softmax; the lanes issue one load each.
    if (lane == 0) {
      mbar_expect_tx(q_full, Q_BYTES);
      for (int hf = 0; hf < NH; ++hf) tma_load_2d(sQ + hf * HALF_BYTES, &map_q, q_full, h * HD + hf * 64, q0 + tile0);
    }
    const int last_block = k_last & ~15;
    const int which = lane / (8 * NH);               // 0: keys, 1: values (lanes beyond have nothing to do)
    const int blk = (lane % (8 * NH)) / NH, hf = lane % NH;
    if (which < 2) {
      // the lanes that load keys and the lanes that load values each follow their own barriers
      const int leader = which * 8 * NH;
      const unsigned group = ((1u << (8 * NH)) - 1u) << leader;
      uint64_t* full = which ? v_full : k_full;
      uint64_t* empty = which ? v_empty : k_empty;
      uint8_t* dst = (which ? sV : sK) + hf * HALF_BYTES + blk * 16 * 128;
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % KV_ST;
        int key0 = (tile_begin + j) * KT + blk * 16;
        if (key0 > last_block) key0 = last_block;            // keys nobody sees: any valid page will do
        const int pg = bt[key0 / a.page];                    // fetched before the wait: its latency is the wait's
        int ok = 1;
        if (lane == leader) {
          ok = mbar_wait(&empty[s], ((j / KV_ST) & 1) ^ 1, a.err, 11) ? 1 : 0;
          if (ok) mbar_expect_tx(&full[s], K_BYTES);
        }
        ok = __shfl_sync(group, ok, leader);
        if (!ok) break;
        const int row = ((pg * 2 + which) * a.Hkv + kvh) * a.page + (key0 % a.page);
        tma_load_2d(dst + s * K_BYTES, &map_kv, &full[s], hf * 64, row);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(QT, KT, 0);
      constexpr uint32_t idesc_pv = umma_idesc(QT, HD, 1);
      bool ok = mbar_wait(q_full, 0, a.err, 12);
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1, ks = j % KV_ST;
        if (!mbar_wait(&k_full[ks], (j / KV_ST) & 1, a.err, 13)) return false;
        if (!mbar_wait(&s_empty[s], ((j >> 1) & 1) ^ 1, a.err, 14)) return false;
        tc_fence_after();
        const uint32_t d = tmem + (uint32_t)(s * KT);
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) {
          const uint64_t dq = umma_desc(smem_u32(sQ + hf * HALF_BYTES));
          const uint64_t dk = umma_desc(smem_u32(sK + ks * K_BYTES + hf * HALF_BYTES));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_f16(d, dq + 2 * kk, dk + 2 * kk, idesc_qk, (hf > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
        umma_commit(&k_empty[ks]);                   // the keys' stage is free once this product has read it
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_qk(j + 1);
        if (!ok) break;
        const int s = j % KV_ST;                     // the stage of this tile's keys and values
        if (!mbar_wait(&v_full[s], (j / KV_ST) & 1, a.err, 16)) break;
        if (!mbar_wait(p_full, j & 1, a.err, 15)) break;
        tc_fence_after();
        // P [128 rows][128 keys] in tensor memory (64 columns of two keys); V [128 keys][HD] MN-major
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
          const uint32_t v_addr = smem_u32(sV + s * K_BYTES + (kk * 16) * 128);
          umma_f16_ts(tmem_pv, tmem_p + (uint32_t)(kk * 8), umma_desc_mn(v_addr, HALF_BYTES), idesc_pv, (kk > 0 || j > 0) ? 1u : 0u);
        }
        umma_commit(pv_full);
        umma_commit(&v_empty[s]);
        umma_commit(p_empty);
      }
    }
  } else {
    // softmax: thread = (query row, share of the tile's keys)
    const int qd = warp & 3;                           // the quarter of tensor memory's lanes this warp may touch
    const int wg = (warp - 2) >> 2;                    // which share of the keys and of the output columns
    const int r = qd * 32 + lane;
    const int row_in_seg = tile0 + r;
    const int hi = row_in_seg < qlen ? pos0 + row_in_seg : -1;
    const int lo = (a.window > 0 && hi - a.window + 1 > 0) ? hi - a.window + 1 : 0;
    const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
    bf16* mx_x = (bf16*)(xchg + qd * 256);
    float* l_x = (float*)(xchg + qd * 256);
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    // A wait that gives up makes the whole warp skip the rest of its work, but not the meetings with
    // its partner warps: those are kept to the end, so that nobody waits at a barrier for ever.
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      const int key_base = (tile_begin + j) * KT + wg * KPT;
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&s_full[s], (j >> 1) & 1, a.err, 17));
      float mx = -INFINITY;
      uint32_t sv[KPT];                                  // this thread's part of the row of S, read once
      const bool all_visible = key_base >= lo && key_base + KPT - 1 <= hi;   // no mask needed in this part
      if (ok) {
        tc_fence_after();
        const uint32_t s_addr = tmem + lane_base + (uint32_t)(s * KT + wg * KPT);
#pragma unroll
        for (int c = 0; c < KPT; c += 32) tmem_ld32(s_addr + c, sv + c);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&s_empty[s]);                     // S[s] may be overwritten by tile j + 2
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
        bf16* slot = mx_x + (j & 1) * (WGS * 32);
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
      // the exponentials first, into registers: nothing here waits for the tensor pipe, so this runs
      // while the product of the tile before is still under way
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
      // P's columns are free, and the output row is at rest, once the previous tile's P.V is done
      ok = __all_sync(0xffffffffu, mbar_wait(p_empty, (j & 1) ^ 1, a.err, 18));
      if (!ok) continue;
      tc_fence_after();
      if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
        // some row of this warp moves its reference: scale this thread's columns of the warp's rows
        // of O (by 1 where nothing moved); the partner warps decide alike, from the same values
#pragma unroll
        for (int c = 0; c < OPT; c += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_pv + lane_base + (uint32_t)(wg * OPT + c), v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
          tmem_st32(tmem_pv + lane_base + (uint32_t)(wg * OPT + c), v);
        }
      }
#pragma unroll
      for (int c = 0; c < KPT; c += 64) tmem_st32(tmem_p + lane_base + (uint32_t)((wg * KPT + c) >> 1), w + (c >> 1));
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (WGS > 1) {
      // the row's sum: every thread's part, added in the same order by all of them.  The barrier
      // first: the maxima of the last two tiles lie in the bytes the sums go to.
      named_barrier(1 + qd, 32 * WGS);
      l_x[wg * 32 + lane] = l;
      named_barrier(1 + qd, 32 * WGS);
      l = 0.f;
#pragma unroll
      for (int w = 0; w < WGS; ++w) l += l_x[w * 32 + lane];
    }
    if (ok && n_tiles > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(pv_full, (n_tiles - 1) & 1, a.err, 20));
      tc_fence_after();
      // every lane takes part in the loads (they are warp-wide); only rows of the segment are stored
      const bool store = ok && row_in_seg < qlen;
      const float inv = store ? 1.f / l : 0.f;
      bf16* orow = a.out + (size_t)(q0 + (store ? row_in_seg : 0)) * a.ld_out + (size_t)h * HD + wg * OPT;
#pragma unroll
      for (int c = 0; c < OPT; c += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_pv + lane_base + (uint32_t)(wg * OPT + c), v);
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
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mkv, const AttnArgs& args, dim3 grid, cudaStream_t st) {
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
  return qv_launch(kernel, grid, dim3(64 + 128 * SOFTMAX_WGS), (size_t)smem, st, mq, mkv, args);
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
  if (S > 65535 || (max_q_len + QT - 1) / QT > 65535) return QV_ERR_TOO_LARGE;
  CUtensorMap mq, mkv;
  if (!make_map(&mq, q, T, H * hd, ld_q, QT)) return QV_ERR_UNSUPPORTED;
  if (!make_map(&mkv, cache, cache_pages * 2 * Hkv * page, hd, hd, 16)) return QV_ERR_UNSUPPORTED;
  AttnArgs a;
  a.out = (bf16*)out; a.seg_q_start = seg_q_start; a.seg_pos0 = seg_pos0; a.block_table = block_table; a.err = err;
  a.ld_out = ld_out; a.max_blocks = max_blocks; a.H = H; a.Hkv = Hkv; a.page = page; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(H, (max_q_len + QT - 1) / QT, S);
  if (hd == 128) return launch<128>(mq, mkv, a, grid, (cudaStream_t)stream);
  return launch<64>(mq, mkv, a, grid, (cudaStream_t)stream);
}
