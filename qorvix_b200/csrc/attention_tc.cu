// Flash attention for prompt portions on the 5th-generation tensor cores (sm_100a), over the
// paged bfloat16 cache: Q.K^T and P.V are tcgen05.mma instructions with their accumulators in
// tensor memory; Q, K and V tiles arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle), the
// keys and values page by page through the request's block table.  Formula and masking are the
// reference's (runtime/src/text_model.cpp:83-114); its CUDA kernel handles one query at a time on
// the CUDA cores (cuda/src/cuda_backend.cu:347-395).
//
// One CTA = 128 query rows of one head, walking 128-key tiles:
//   warp 0        TMA: Q once, then K and V tiles into a two-stage ring
//   warp 1        MMA: S[j] = Q K_j^T into one of two S buffers in tensor memory (so that S[j+1] is
//                 computed while the softmax of tile j runs), then PV_j = P_j V_j
//   warps 2..5    softmax: thread r owns query row r: reads S from tensor memory twice (row maximum,
//                 then exponentials), writes P as bfloat16 into swizzled shared memory for the next
//                 MMA, and keeps the output row in registers: O = (O + PV_{j-1}) * exp2(m_{j-1} - m_j)
// Softmax statistics, rescaling and the output sum are float32.  Every mbarrier wait is bounded
// and reports through *err instead of hanging.
#include "common.cuh"

#ifndef QV_P_TMEM
#define QV_P_TMEM 1      // P goes to the P.V product through tensor memory (1) or shared memory (0)
#endif
#ifndef QV_O_TMEM
#define QV_O_TMEM 1      // the output row accumulates in tensor memory across key tiles (1) or in registers (0)
#endif
#define KV_ST (QV_P_TMEM ? 3 : 2)   // stages of keys and values in shared memory (P's buffer, when there is one, takes a stage's room)
#define RESCALE_STEP 8.0f   // with QV_O_TMEM: the reference maximum of a row moves only when it grew by more than 2^8
#include <cuda.h>

#define QT 128             // query rows per CTA
#define KT 128             // keys per tile
#define WAIT_LIMIT (1u << 22)

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err, int code) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  atomicExch(err, code);
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// MN-major operand (V: head dims contiguous), 128-byte swizzle: 64 elements of N per 128-byte row,
// rows are consecutive k (keys) 128 bytes apart, 8-key groups 1024 bytes apart (SBO), the next 64
// elements of N `lbo_bytes` further (LBO).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo_bytes) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
// the same with the A operand in tensor memory (row = lane, two bfloat16 of consecutive k per column)
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 2^x for x <= 0 on the special-function unit (results below the normal range flush to zero; P is
// rounded to bfloat16 right after, so the approximation's last bits do not matter)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&h;
}

struct AttnArgs {
  bf16* out;
  const int* seg_q_start;
  const int* seg_pos0;
  const int* block_table;
  int* err;
  int ld_out, max_blocks, H, Hkv, page, window;
  float scale_log2;
};

template <int HD>
__global__ void __launch_bounds__(192) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                              const __grid_constant__ CUtensorMap map_kv, const AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int NH = HD / 64;                        // 64-element halves of the head
  constexpr int Q_BYTES = QT * HD * 2;               // [NH][128 rows][64]
  constexpr int K_BYTES = KT * HD * 2;               // [NH][128 keys][64]
  constexpr int P_BYTES = QT * KT * 2;               // [2][128 rows][64 keys]
  constexpr int HALF_BYTES = 128 * 128;              // one [128][64] bf16 tile
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = base;
  uint8_t* sK = sQ + Q_BYTES;                        // 2 stages
  uint8_t* sV = sK + KV_ST * K_BYTES;                // KV_ST stages each
  uint8_t* sP = sV + KV_ST * K_BYTES;                // only without QV_P_TMEM
  uint64_t* bars = (uint64_t*)(sP + (QV_P_TMEM ? 0 : P_BYTES));
  uint64_t* q_full = bars;                           // 1
  uint64_t* kv_full = bars + 13;                     // KV_ST
  uint64_t* kv_empty = bars + 16;                    // KV_ST
  uint64_t* s_full = bars + 5;                       // 2
  uint64_t* s_empty = bars + 7;                      // 2
  uint64_t* p_full = bars + 9;
  uint64_t* p_empty = bars + 10;
  uint64_t* pv_full = bars + 11;
  uint64_t* pv_empty = bars + 12;
  uint32_t* tmem_slot = (uint32_t*)(bars + 19);

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
    for (int i = 0; i < KV_ST; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 128); }
    mbar_init(p_full, 128); mbar_init(p_empty, 1); mbar_init(pv_full, 1); mbar_init(pv_empty, 128);
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
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_pv = tmem + 256;
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
    const int which = lane / (8 * NH);               // 0: keys, 1: values
    const int blk = (lane % (8 * NH)) / NH, hf = lane % NH;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j % KV_ST;
      if (lane == 0) {
        ok = mbar_wait(&kv_empty[s], ((j / KV_ST) & 1) ^ 1, a.err, 11);
        if (ok) mbar_expect_tx(&kv_full[s], 2 * K_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (which < 2) {
        int key0 = (tile_begin + j) * KT + blk * 16;
        if (key0 > last_block) key0 = last_block;            // keys nobody sees: any valid page will do
        const int row = ((bt[key0 / a.page] * 2 + which) * a.Hkv + kvh) * a.page + (key0 % a.page);
        tma_load_2d((which ? sV : sK) + s * K_BYTES + hf * HALF_BYTES + blk * 16 * 128, &map_kv, &kv_full[s], hf * 64, row);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = idesc_f16(QT, KT, 0);
      constexpr uint32_t idesc_pv = idesc_f16(QT, HD, 1);
      bool ok = mbar_wait(q_full, 0, a.err, 12);
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1, ks = j % KV_ST;
        if (!mbar_wait(&kv_full[ks], (j / KV_ST) & 1, a.err, 13)) return false;
        if (!mbar_wait(&s_empty[s], ((j >> 1) & 1) ^ 1, a.err, 14)) return false;
        tc_fence_after();
        const uint32_t d = tmem + (uint32_t)(s * KT);
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) {
          const uint64_t dq = desc_kmajor(smem_u32(sQ + hf * HALF_BYTES));
          const uint64_t dk = desc_kmajor(smem_u32(sK + ks * K_BYTES + hf * HALF_BYTES));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma(d, dq + 2 * kk, dk + 2 * kk, idesc_qk, (hf > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_qk(j + 1);
        if (!ok) break;
        const int s = j % KV_ST;                     // the stage of this tile's keys and values
        if (!mbar_wait(p_full, j & 1, a.err, 15)) break;
#if !QV_O_TMEM
        if (!mbar_wait(pv_empty, (j & 1) ^ 1, a.err, 16)) break;
#endif
        tc_fence_after();
#if QV_P_TMEM
        // P [128 rows][128 keys] in tensor memory (64 columns of two keys); V [128 keys][HD] MN-major
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
          const uint32_t v_addr = smem_u32(sV + s * K_BYTES + (kk * 16) * 128);
          umma_ts(tmem_pv, tmem_p + (uint32_t)(kk * 8), desc_mnmajor(v_addr, HALF_BYTES), idesc_pv, (kk > 0 || (QV_O_TMEM && j > 0)) ? 1u : 0u);
        }
#else
        // P [128 rows][128 keys] as two K-major halves of 64 keys; V [128 keys][HD] MN-major
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) {
          const uint64_t dp = desc_kmajor(smem_u32(sP + kh * HALF_BYTES));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t v_addr = smem_u32(sV + s * K_BYTES + (kh * 64 + kk * 16) * 128);
            umma(tmem_pv, dp + 2 * kk, desc_mnmajor(v_addr, HALF_BYTES), idesc_pv, (kh > 0 || kk > 0) ? 1u : 0u);
          }
        }
#endif
        umma_commit(pv_full);
        umma_commit(&kv_empty[s]);
        umma_commit(p_empty);
      }
    }
  } else {
    // softmax: thread = query row
#if QV_O_TMEM && QV_P_TMEM
    // The output row lives in tensor memory and the P.V products accumulate into it; a row's
    // reference maximum moves only when the true maximum has grown by more than 2^RESCALE_STEP
    // (then the row in tensor memory is scaled down once), so P may reach 2^RESCALE_STEP and most
    // tiles need neither a second pass over S nor any work on O.
    const int qd = warp & 3;
    const int r = qd * 32 + lane;
    const int row_in_seg = tile0 + r;
    const int hi = row_in_seg < qlen ? pos0 + row_in_seg : -1;
    const int lo = (a.window > 0 && hi - a.window + 1 > 0) ? hi - a.window + 1 : 0;
    const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      const int key_base = (tile_begin + j) * KT;
      ok = mbar_wait(&s_full[s], (j >> 1) & 1, a.err, 17);
      tc_fence_after();
      const uint32_t s_addr = tmem + lane_base + (uint32_t)(s * KT);
      uint32_t sv[KT];                                   // this row of S, read once
#pragma unroll
      for (int c = 0; c < KT; c += 32) tmem_ld32(s_addr + c, sv + c);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&s_empty[s]);                       // S[s] may be overwritten by tile j + 2
      const bool all_visible = key_base >= lo && key_base + KT - 1 <= hi;   // no mask needed in this tile
      float mx = -INFINITY;
      if (all_visible) {
#pragma unroll
        for (int i = 0; i < KT; ++i) mx = fmaxf(mx, __uint_as_float(sv[i]));
      } else {
#pragma unroll
        for (int i = 0; i < KT; ++i) {
          const int key = key_base + i;
          if (key >= lo && key <= hi) mx = fmaxf(mx, __uint_as_float(sv[i]));
        }
      }
      mx *= a.scale_log2;                              // the scale is positive: max commutes with it
      float corr = 1.f;
      if (mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY)) {
        corr = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - mx);
        m_ref = mx;
      }
      // P's columns are free, and the output row is at rest, once the previous tile's P.V is done
      if (ok) ok = mbar_wait(p_empty, (j & 1) ^ 1, a.err, 18);
      tc_fence_after();
      if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
        // some row of this warp moves its reference: scale the warp's rows of O (by 1 where nothing moved)
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_pv + lane_base + c, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
          tmem_st32(tmem_pv + lane_base + c, v);
        }
      }
      l *= corr;
      float sum = 0.f;
      const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
#pragma unroll
      for (int c = 0; c < KT; c += 64) {
        uint32_t w[32];
        if (all_visible) {                             // most tiles: no mask, two instructions per score
#pragma unroll
          for (int i = 0; i < 64; i += 2) {
            const float e0 = fast_exp2(fmaf(__uint_as_float(sv[c + i]), a.scale_log2, neg_m));
            const float e1 = fast_exp2(fmaf(__uint_as_float(sv[c + i + 1]), a.scale_log2, neg_m));
            sum += e0 + e1;
            w[i >> 1] = pack2(e0, e1);
          }
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
            w[i >> 1] = pack2(e[0], e[1]);
          }
        }
        tmem_st32(tmem_p + lane_base + (uint32_t)(c >> 1), w);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full);
      l += sum;
    }
    if (ok && n_tiles > 0) {
      ok = mbar_wait(pv_full, (n_tiles - 1) & 1, a.err, 20);
      tc_fence_after();
      // every lane takes part in the loads (they are warp-wide); only rows of the segment are stored
      const bool store = ok && row_in_seg < qlen;
      const float inv = store ? 1.f / l : 0.f;
      bf16* orow = a.out + (size_t)(q0 + (store ? row_in_seg : 0)) * a.ld_out + (size_t)h * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_pv + lane_base + c, v);
        tmem_wait_ld();
        if (store) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *(uint4*)(orow + c + i) = make_uint4(pack2(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv),
                                                 pack2(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv),
                                                 pack2(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv),
                                                 pack2(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv));
        }
      }
    }
    tc_fence_before();
  }
#else
    const int qd = warp & 3;
    const int r = qd * 32 + lane;
    const int row_in_seg = tile0 + r;
    const int hi = row_in_seg < qlen ? pos0 + row_in_seg : -1;
    const int lo = (a.window > 0 && hi - a.window + 1 > 0) ? hi - a.window + 1 : 0;
    const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      const int key_base = (tile_begin + j) * KT;
      ok = mbar_wait(&s_full[s], (j >> 1) & 1, a.err, 17);
      tc_fence_after();
      const uint32_t s_addr = tmem + lane_base + (uint32_t)(s * KT);
      // pass 1: row maximum of the visible, scaled scores
      float mx = -INFINITY;
      const bool all_visible = key_base >= lo && key_base + KT - 1 <= hi;   // no mask needed in this tile
#pragma unroll 1
      for (int c = 0; c < KT; c += 64) {
        uint32_t v[64];
        tmem_ld32(s_addr + c, v);
        tmem_ld32(s_addr + c + 32, v + 32);
        tmem_wait_ld();
        if (all_visible) {
#pragma unroll
          for (int i = 0; i < 64; ++i) mx = fmaxf(mx, __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const int key = key_base + c + i;
            if (key >= lo && key <= hi) mx = fmaxf(mx, __uint_as_float(v[i]));
          }
        }
      }
      mx *= a.scale_log2;                              // the scale is positive: max commutes with it
      const float m_new = fmaxf(m, mx);
      const float corr = (m_new == -INFINITY) ? 1.f : exp2f(m - m_new);
      // the P buffer is free once the previous tile's P.V has read it
      if (ok) ok = mbar_wait(p_empty, (j & 1) ^ 1, a.err, 18);
      // pass 2: exponentials, row sum, P into shared memory (K-major, 128-byte swizzle)
      float sum = 0.f;
      const float neg_m = -m_new;
#pragma unroll 1
      for (int c = 0; c < KT; c += 64) {
        uint32_t v[64];
        tmem_ld32(s_addr + c, v);
        tmem_ld32(s_addr + c + 32, v + 32);
        tmem_wait_ld();
        uint32_t w[32];
        if (all_visible) {                             // most tiles: no mask, two instructions per score
#pragma unroll
          for (int i = 0; i < 64; i += 2) {
            const float e0 = fast_exp2(fmaf(__uint_as_float(v[i]), a.scale_log2, neg_m));
            const float e1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), a.scale_log2, neg_m));
            sum += e0 + e1;
            w[i >> 1] = pack2(e0, e1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 64; i += 2) {
            float e[2];
#pragma unroll
            for (int x = 0; x < 2; ++x) {
              const int key = key_base + c + i + x;
              e[x] = (key >= lo && key <= hi) ? fast_exp2(fmaf(__uint_as_float(v[i + x]), a.scale_log2, neg_m)) : 0.f;
            }
            sum += e[0] + e[1];
            w[i >> 1] = pack2(e[0], e[1]);
          }
        }
#if QV_P_TMEM
        // 64 keys = 32 columns of this row's P in tensor memory
        tmem_st32(tmem_p + lane_base + (uint32_t)(c >> 1), w);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&s_empty[s]);                       // S[s] may be overwritten by tile j + 2
      mbar_arrive(p_full);
#else
        // 64 keys = the 8 chunks of 16 bytes of this row in half (c / 64)
        uint8_t* prow = sP + (c >> 6) * HALF_BYTES + r * 128;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          *(uint4*)(prow + ((k ^ (r & 7)) << 4)) = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
      }
      tc_fence_before();
      mbar_arrive(&s_empty[s]);                       // S[s] may be overwritten by tile j + 2
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(p_full);
#endif
      // fold in the previous tile's P.V, then rescale to the new maximum
      if (j > 0) {
        if (ok) ok = mbar_wait(pv_full, (j - 1) & 1, a.err, 19);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_pv + lane_base + c, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c + i] = (o[c + i] + __uint_as_float(v[i])) * corr;
        }
        tc_fence_before();
        mbar_arrive(pv_empty);
      }
      l = l * corr + sum;
      m = m_new;
    }
    if (ok && n_tiles > 0) {
      ok = mbar_wait(pv_full, (n_tiles - 1) & 1, a.err, 20);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_pv + lane_base + c, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c + i] += __uint_as_float(v[i]);
      }
    }
    if (ok && row_in_seg < qlen) {
      const float inv = 1.f / l;
      bf16* orow = a.out + (size_t)(q0 + row_in_seg) * a.ld_out + (size_t)h * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 8)
        *(uint4*)(orow + c) = make_uint4(pack2(o[c] * inv, o[c + 1] * inv), pack2(o[c + 2] * inv, o[c + 3] * inv),
                                         pack2(o[c + 4] * inv, o[c + 5] * inv), pack2(o[c + 6] * inv, o[c + 7] * inv));
    }
    tc_fence_before();
  }
#endif
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}
bool make_map(CUtensorMap* map, const void* ptr, long long rows, int cols, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mkv, const AttnArgs& args, dim3 grid, cudaStream_t st) {
  constexpr int smem = QT * HD * 2 + 2 * KV_ST * KT * HD * 2 + (QV_P_TMEM ? 0 : QT * KT * 2) + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return qv_launch(attn_prefill_tc_kernel<HD>, grid, dim3(192), (size_t)smem, st, mq, mkv, args);
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
