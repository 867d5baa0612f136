// C[M,N] = A[M,K] * W[N,K]^T in bfloat16 on the 5th-generation tensor cores (sm_100a):
// operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), products
// issued by one thread with tcgen05.mma, float32 accumulators in tensor memory, read back with
// tcgen05.ld for the epilogue.  The reference multiplies one row at a time on the CUDA cores
// (cuda/src/cuda_backend.cu:291-312); this kernel is its replacement for both phases:
//
//   * many tokens (prefill): the token rows are the 128-row MMA operand, 256 (or 128) weight
//     rows the other; a persistent kernel, one CTA per SM walking over the tiles, with the
//     accumulator double-buffered in tensor memory so that one tile's epilogue overlaps the next
//     tile's main loop.  The epilogue may apply SwiGLU (gate/up projection) or rotate the query and
//     key heads and write keys and values into the paged cache (QKV projection).  A product with
//     fewer tiles than SMs and a long K shares its tiles' k blocks between all SMs (partial sums
//     through a float32 workspace, added in a fixed order).
//   * few tokens (decode, M <= 64): operands are swapped.  128 weight rows are the 128-row MMA
//     operand and the tokens (padded to 16/32/64) the narrow one, so every weight byte is
//     streamed from HBM exactly once through a deep TMA ring.  Matrices with few row tiles are
//     also split along K so that enough CTAs pull from HBM at once; the CTAs of one tile form a
//     thread-block cluster, leave their partial sums in shared memory, and the first CTA adds
//     them through distributed shared memory in a fixed order (split 0, 1, 2, ...).
//
// Every wait on an mbarrier is bounded; when one gives up it records a code in *err and the
// CTA winds down (tensor memory is freed) instead of hanging the device.
#include "tc_common.cuh"

#define A_TILE_BYTES (BM * BK * 2)

namespace {

struct GemmArgs {
  void* C;             // output [tokens, features], row stride ldc
  int* err;
  int rows_wide;       // rows of the operand that feeds the 128-row side
  int rows_narrow;     // rows of the other operand
  int K;
  int ldc;
  int kblocks_per_split;
  int splits;
  const uint8_t* packed;   // the weight matrix as 16 KB tiles (see qv_pack_weight_tiles), or null
  int bn;                  // persistent kernel: columns of a tile (a multiple of 16, at most its BN)
};

// What the fused rotary epilogue of the QKV product needs: C's columns are H query heads, Hkv key
// heads and Hkv value heads of hd dims; query and key heads are rotated (all hd dims, in split-half
// pairs) by the angles of the token's position, keys and values go to the token's slot in its page.
struct RopeArgs {
  const float2* cos_sin = nullptr;   // [table_rows][hd / 2] of (cos, sin); null: no fused rotation
  const int* tok_pos = nullptr;
  const int* tok_seg = nullptr;
  const int* block_table = nullptr;  // [segments][max_blocks]
  bf16* cache = nullptr;             // the layer's pages: [page][2][Hkv][page_size][hd]
  int table_rows = 0, max_blocks = 0, H = 0, Hkv = 0, hd = 0, page_size = 0;
};

// The norm that follows or precedes a product of few tokens, folded into it (few-token kernel only).
// After an output projection: the product is added into the float32 residual stream, C gets the
// updated stream times the next norm's weight (bfloat16), and ssq_out the sums of squares of the
// updated stream per tile of 128 features, [tiles][64 tokens].  Before a projection that reads such
// a C: each token's sums are scaled by rsqrt(mean of squares + eps), which completes the RMS norm.
struct NormArgs {
  float* residual = nullptr;       // [tokens][ld_res]; null: the product is stored as it is
  const float* norm_w = nullptr;
  float* ssq_out = nullptr;
  const float* ssq_in = nullptr;   // null: no scaling
  int ld_res = 0, tiles_in = 0;
  float inv_d = 0.f, eps = 0.f;
};

// Few tokens.  BN: columns of the accumulator (token rows per tile, padded).  The wide operand is
// the weight matrix (features) and the narrow one the tokens, so the tile is C^T.
// SWIGLU: the weight rows come in groups of 32 (16 gate rows, then the 16 up rows of the same
// features); the epilogue writes silu(gate) * up, so C has half as many features as W has rows.
// bfloat16 output: the fast exponential's error (a few float32 ulp) vanishes in the rounding
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

template <int BN, int STAGES, typename TC, bool SWIGLU>
__global__ void __launch_bounds__(192) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_wide,
                                                      const __grid_constant__ CUtensorMap map_narrow,
                                                      const GemmArgs args, const NormArgs norm) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(tiles + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* accum = empty + STAGES;
  uint32_t* tmem_slot = (uint32_t*)(accum + 1);
  int* ok_slots = (int*)(tmem_slot + 1);  // one per epilogue warp
  float* rs_s = (float*)(ok_slots + 4);   // [64] a token's rsqrt(mean of squares + eps), with NormArgs::ssq_in
  float* rs_part = rs_s + 64;             // [128] the threads' shares of the sums behind rs_s

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;   // known to be uniform
  const int wide0 = blockIdx.x * BM;
  const int narrow0 = blockIdx.y * BN;
  const int split = blockIdx.z;
  const int total_kb = (args.K + BK - 1) / BK;
  const int kb0 = split * args.kblocks_per_split;
  int num_kb = total_kb - kb0;
  if (num_kb > args.kblocks_per_split) num_kb = args.kblocks_per_split;
  if (num_kb < 0) num_kb = 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(accum, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  // NormArgs::residual: the stream's values for the first 16 tokens and the norm's weight, fetched by
  // the first CTA's epilogue threads while the main loop runs
  float stream0[16];
  float norm_w0 = 0.f;

  if (warp == 0) {
    {
      // (the whole warp walks the loop and waits, an elected lane requests: see the MMA warp)
      const bool leader = elect_one();
      // Weights are never written by a kernel, so the first stages' weight tiles are requested
      // before waiting for the kernel ahead in the stream; the activation tiles after.
      const CUtensorMap* w_map = &map_wide;
      const CUtensorMap* x_map = &map_narrow;
      const int w_row0 = wide0, x_row0 = narrow0;
      const int w_off = 0, x_off = A_BYTES;
      const int pre = num_kb < STAGES ? num_kb : STAGES;
      // a packed weight matrix is read tile by tile with contiguous 16 KB copies; its tiles are 128
      // rows, so the weight side of this kernel's tile must be 128 rows too (the host sees to that)
      const uint8_t* wp = args.packed ? args.packed + ((size_t)blockIdx.x * total_kb + kb0) * (size_t)A_BYTES : nullptr;
      if (leader) {
        for (int kb = 0; kb < pre; ++kb) {
          mbar_expect_tx(&full[kb], STAGE_BYTES);
          if (wp) bulk_load_1d(tiles + kb * STAGE_BYTES + w_off, wp + (size_t)kb * A_BYTES, &full[kb], A_BYTES);
          else tma_load_2d(tiles + kb * STAGE_BYTES + w_off, w_map, &full[kb], (kb0 + kb) * BK, w_row0);
        }
      }
      __syncwarp();
      pdl_wait();
      if (leader) {
        for (int kb = 0; kb < pre; ++kb)
          tma_load_2d(tiles + kb * STAGE_BYTES + x_off, x_map, &full[kb], (kb0 + kb) * BK, x_row0);
      }
      __syncwarp();
      for (int kb = pre; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, args.err, 1)) break;
        if (leader) {
          mbar_expect_tx(&full[s], STAGE_BYTES);
          uint8_t* a = tiles + s * STAGE_BYTES;
          if (wp) bulk_load_1d(a + w_off, wp + (size_t)kb * A_BYTES, &full[s], A_BYTES);
          else tma_load_2d(a + w_off, w_map, &full[s], (kb0 + kb) * BK, w_row0);
          tma_load_2d(a + x_off, x_map, &full[s], (kb0 + kb) * BK, x_row0);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    {
      // the whole warp walks the loop and waits; one elected lane issues (its operands then stay in uniform registers)
      const bool leader = elect_one();
      constexpr uint32_t idesc = umma_idesc(BM, BN);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        ok = mbar_wait(&full[s], ph, args.err, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES);
        const uint64_t da = umma_desc(a_addr), db = umma_desc(a_addr + A_BYTES);
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)    // 16 k elements = 32 bytes = 2 descriptor units
            umma_f16(tmem_base, da + 2 * kk, db + 2 * kk, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&empty[s]);                  // frees the stage when these MMAs have read it
        }
        __syncwarp();
      }
      if (leader) umma_commit(accum);              // accumulator complete (or nothing was issued)
      __syncwarp();
    }
  } else {
    // epilogue: warps 2..5 own TMEM lanes 32*(warp%4) .. +31
    pdl_wait();                 // C may still be in use by the kernel ahead
    const int q = warp & 3;
    if (norm.ssq_in != nullptr && (args.splits == 1 || split == 0)) {
      // While the main loop runs: each token's scale from the sums of squares the kernel ahead left.
      // The 128 threads share the loads (128 / BN threads a token, each every (128 / BN)-th tile, four
      // loads in flight a thread), then one thread a token adds the parts in a fixed order.
      constexpr int PER = 128 / BN;
      const int te = q * 32 + lane;
      const int tok = te % BN, part = te / BN;
      const int t = narrow0 + tok;
      float ss = 0.f;
      if (t < args.rows_narrow) {
        for (int k = part; k < norm.tiles_in; k += 4 * PER) {
          float v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) v[u] = k + u * PER < norm.tiles_in ? norm.ssq_in[(k + u * PER) * 64 + t] : 0.f;
          ss += (v[0] + v[1]) + (v[2] + v[3]);
        }
      }
      rs_part[te] = ss;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (te < BN) {
        float tot = 0.f;
#pragma unroll
        for (int u = 0; u < PER; ++u) tot += rs_part[u * BN + te];
        rs_s[te] = rsqrtf(tot * norm.inv_d + norm.eps);
      }
    }
    if (norm.residual != nullptr && split == 0) {
      const int wr = wide0 + q * 32 + lane;
      const bool v = wr < args.rows_wide;
      norm_w0 = v ? norm.norm_w[wr] : 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j)
        stream0[j] = (v && narrow0 + j < args.rows_narrow) ? norm.residual[(size_t)(narrow0 + j) * norm.ld_res + wr] : 0.f;
    }
    // one lane per warp polls; the four warps then agree, so that either all of them take the
    // barriers below or none does
    int ok_i = 1;
    if (lane == 0) {
      ok_i = mbar_wait(accum, 0, args.err, 3) ? 1 : 0;
      ok_slots[q] = ok_i;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const bool ok = ok_slots[0] && ok_slots[1] && ok_slots[2] && ok_slots[3];
    tc_fence_after();
    const int wide_row = wide0 + q * 32 + lane;          // row of the wide operand this thread holds
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
    TC* C = (TC*)args.C;
    if (ok && num_kb > 0) {
      // thread = feature wide_row; columns = tokens narrow0 + c
      const bool frow = wide_row < args.rows_wide;
      const int ntok = args.rows_narrow;
      if (args.splits == 1) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_wait_ld();
          if (SWIGLU) {
            // lanes 0..15 hold gate rows, lanes 16..31 the up rows of the same features
            const int feat = ((wide0 + q * 32) >> 1) + (lane & 15);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float mine = __uint_as_float(r[j]) * (norm.ssq_in ? rs_s[c0 + j] : 1.f);
              const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
              const int t = narrow0 + c0 + j;
              if (lane < 16 && frow && t < ntok) store_out<TC>(C + (size_t)t * args.ldc + feat, silu_mul(mine, other));
            }
          } else if (frow) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = narrow0 + c0 + j;
              if (t < ntok) store_out<TC>(C + (size_t)t * args.ldc + wide_row, __uint_as_float(r[j]) * (norm.ssq_in ? rs_s[c0 + j] : 1.f));
            }
          }
        }
      } else {
        // split-K: this CTA's partial sums go to its own shared memory (the stage ring is free
        // now), column-major so that a warp's 32 rows are 32 consecutive floats; the cluster's
        // first CTA adds them up below
        float* red = (float*)tiles;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) red[(c0 + j) * BM + q * 32 + lane] = __uint_as_float(r[j]);
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (args.splits > 1) {
    // The CTAs of one tile (one per split) form a cluster.  After the cluster barrier every
    // partial tile is visible through distributed shared memory; the first CTA adds them in
    // split order 0, 1, 2, ... and stores the result, and a second barrier keeps the others'
    // shared memory alive until it has.
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    if (split == 0 && warp >= 2) {
      const int row = (warp & 3) * 32 + lane;
      const int wide_row = wide0 + row;
      const int ntok = args.rows_narrow;
      const float* red = (const float*)tiles;
      const uint32_t red_addr = smem_u32(red);
      TC* C = (TC*)args.C;
      const bool valid = wide_row < args.rows_wide;
      const bool to_stream = norm.residual != nullptr;        // add into the residual stream, hand on the next norm's input
      float* part_s = (float*)tiles + BN * BM;                // after this CTA's own partial sums
      const float wn = norm_w0;
      if (valid || to_stream) {
        for (int j0 = 0; j0 < BN && narrow0 + j0 < ntok; j0 += 16) {
          float acc[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] = valid ? red[(j0 + j) * BM + row] : 0.f;
          // the other CTAs' partial sums, three CTAs' worth of loads in flight together (one trip
          // through distributed shared memory for up to four splits), added in split order
          for (int s0 = 1; valid && s0 < args.splits; s0 += 3) {
            float v[3][16];
#pragma unroll
            for (int q = 0; q < 3; ++q) {
              uint32_t remote = 0;
              if (s0 + q < args.splits)
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(red_addr + (uint32_t)((j0 * BM + row) * 4)), "r"(s0 + q));
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                v[q][j] = 0.f;
                if (s0 + q < args.splits && narrow0 + j0 + j < ntok)
                  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[q][j]) : "r"(remote + (uint32_t)(j * BM * 4)) : "memory");
              }
            }
#pragma unroll
            for (int q = 0; q < 3; ++q)
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[j] += v[q][j];
          }
          if (norm.ssq_in != nullptr) {
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] *= rs_s[j0 + j];
          }
          if (to_stream) {
            float rv[16];
            if (j0 == 0) {
#pragma unroll
              for (int j = 0; j < 16; ++j) rv[j] = stream0[j];
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                rv[j] = (valid && narrow0 + j0 + j < ntok) ? norm.residual[(size_t)(narrow0 + j0 + j) * norm.ld_res + wide_row] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = narrow0 + j0 + j;
              float sq = 0.f;
              if (valid && t < ntok) {
                const float r = rv[j] + acc[j];
                norm.residual[(size_t)t * norm.ld_res + wide_row] = r;
                store_out<TC>(C + (size_t)t * args.ldc + wide_row, r * wn);
                sq = r * r;
              }
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
              if (lane == 0) part_s[(warp & 3) * BN + j0 + j] = sq;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (narrow0 + j0 + j < ntok) store_out<TC>(C + (size_t)(narrow0 + j0 + j) * args.ldc + wide_row, acc[j]);
          }
        }
      }
      if (to_stream) {
        // the tile's sum of squares per token, the four warps' parts added in a fixed order
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int te = (warp & 3) * 32 + lane;
        if (te < BN && narrow0 + te < ntok)
          norm.ssq_out[(size_t)blockIdx.x * 64 + narrow0 + te] = part_s[te] + part_s[BN + te] + part_s[2 * BN + te] + part_s[3 * BN + te];
      }
    }
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// One row's 32 accumulator columns from `col` on go to C: as they are (the first `ncols` of them),
// or, with the fused activation, as the 16 values silu(gate) * up of the features col/2 ...
template <typename TC, bool SWIGLU>
__device__ __forceinline__ void store_chunk(TC* C, int ldc, int row, int col, int ncols, const uint32_t* r) {
  if (SWIGLU) {
    TC* dst = C + (size_t)row * ldc + (col >> 1);
    float a[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) a[j] = silu_mul(__uint_as_float(r[j]), __uint_as_float(r[16 + j]));
    if (sizeof(TC) == 2 && (((uintptr_t)dst) & 15) == 0) {
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = pack2_bf16(a[2 * j], a[2 * j + 1]);
      ((uint4*)dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
      ((uint4*)dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) store_out<TC>(dst + j, a[j]);
    }
  } else {
    TC* dst = C + (size_t)row * ldc + col;
    if (sizeof(TC) == 2 && ncols >= 32 && (((uintptr_t)dst) & 15) == 0) {
      uint4* d4 = (uint4*)dst;
#pragma unroll
      for (int v = 0; v < 4; ++v)
        d4[v] = make_uint4(pack2_bf16(__uint_as_float(r[v * 8]), __uint_as_float(r[v * 8 + 1])),
                           pack2_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3])),
                           pack2_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5])),
                           pack2_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7])));
    } else if (sizeof(TC) == 4 && ncols >= 32 && (((uintptr_t)dst) & 15) == 0) {
      float4* d4 = (float4*)dst;
#pragma unroll
      for (int v = 0; v < 8; ++v)
        d4[v] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
    } else {
      for (int j = 0; j < 32 && j < ncols; ++j) store_out<TC>(dst + j, __uint_as_float(r[j]));
    }
  }
}

// The fused rotary epilogue for one token row of a tile: heads of hd (64 or 128) columns from column
// n0 of C.  Every thread of the warp runs the tensor-memory loads; only rows of real tokens store.
template <int HD>
__device__ __forceinline__ void rope_store_row(const RopeArgs& ra, bf16* C, int ldc, uint32_t taddr, int row, bool live,
                                               int n0, int bn, int N) {
  constexpr int HALF = HD / 2;
  const float2* cs = nullptr;
  bf16* kdst = nullptr;
  if (live) {
    const int pos = ra.tok_pos[row];
    cs = ra.cos_sin + (size_t)(pos < ra.table_rows ? pos : ra.table_rows - 1) * HALF;
    const int pg = ra.block_table[(size_t)ra.tok_seg[row] * ra.max_blocks + pos / ra.page_size];
    kdst = ra.cache + (size_t)pg * ((size_t)2 * ra.Hkv * ra.page_size * HD) + (size_t)(pos % ra.page_size) * HD;
  }
#pragma unroll 1
  for (int h0 = 0; h0 < bn && n0 + h0 < N; h0 += HD) {
    const int head = (n0 + h0) / HD;
    if (head < ra.H + ra.Hkv) {
      bf16* dst = nullptr;
      if (live) dst = head < ra.H ? C + (size_t)row * ldc + (size_t)head * HD : kdst + (size_t)(head - ra.H) * ra.page_size * HD;
#pragma unroll 1
      for (int c = 0; c < HALF; c += 32) {
        uint32_t lo[32], hi[32];
        tmem_ld32(taddr + h0 + c, lo);
        tmem_ld32(taddr + h0 + HALF + c, hi);
        tmem_wait_ld();
        if (!live) continue;
        uint32_t olo[16], ohi[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float4 t = *(const float4*)(cs + c + i);     // (cos, sin) of two neighbouring pairs
          const float a0 = __uint_as_float(lo[i]), a1 = __uint_as_float(lo[i + 1]);
          const float b0 = __uint_as_float(hi[i]), b1 = __uint_as_float(hi[i + 1]);
          olo[i >> 1] = pack2_bf16(a0 * t.x - b0 * t.y, a1 * t.z - b1 * t.w);
          ohi[i >> 1] = pack2_bf16(a0 * t.y + b0 * t.x, a1 * t.w + b1 * t.z);
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          ((uint4*)(dst + c))[v] = make_uint4(olo[4 * v], olo[4 * v + 1], olo[4 * v + 2], olo[4 * v + 3]);
          ((uint4*)(dst + HALF + c))[v] = make_uint4(ohi[4 * v], ohi[4 * v + 1], ohi[4 * v + 2], ohi[4 * v + 3]);
        }
      }
    } else {
      bf16* dst = nullptr;
      if (live) dst = kdst + (size_t)ra.Hkv * ra.page_size * HD + (size_t)(head - ra.H - ra.Hkv) * ra.page_size * HD;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + h0 + c, r);
        tmem_wait_ld();
        if (!live) continue;
#pragma unroll
        for (int v = 0; v < 4; ++v)
          ((uint4*)(dst + c))[v] = make_uint4(pack2_bf16(__uint_as_float(r[v * 8]), __uint_as_float(r[v * 8 + 1])),
                                              pack2_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3])),
                                              pack2_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5])),
                                              pack2_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7])));
      }
    }
  }
}

// ---------------------------------------------------------------- many tokens: persistent kernel
// One CTA per SM; tiles go round the CTAs (tile = blockIdx.x, + gridDim.x, ...; token tiles fastest, so
// that CTAs running at the same time share a weight tile in L2).  A product with fewer tiles than SMs
// (a few hundred tokens times a narrow weight matrix) would leave SMs idle and pay one CTA's whole walk
// along K; there the tiles are shared: their k blocks, tile by tile, are cut into equal contiguous
// shares, one per SM.  A share usually begins inside one tile and ends inside the next.  The CTA that
// has a tile's first k blocks owns the tile; a CTA that has only later k blocks of it leaves its sums
// (float32, from tensor memory) in its slot of a workspace and raises its flag; the owner waits for
// the flags of the CTAs after it (they did that work first of all, while the owner did its own part),
// adds their sums into its accumulator in tensor memory, in CTA order, and runs the epilogue.
// The accumulator is double-buffered in tensor memory (2 x BN columns): while the four epilogue
// warps drain one piece of work, the MMA warp already accumulates the next, and the TMA warp runs
// ahead of both through the shared-memory ring.
struct Segment {
  int tile, kb0, kb1;                                // k blocks [kb0, kb1) of a tile
};
template <bool SHARED>
struct Share {                                       // a CTA's work: a run of k-block units of the shared tiles, or whole tiles
  long long u, end;
  int num_kb, next_tile, stride, total_tiles;
  __device__ __forceinline__ Share(int cta, int ctas, int tiles, int kbs) {
    const long long units = SHARED ? (long long)tiles * kbs : 0;
    u = units * cta / ctas;
    end = units * (cta + 1) / ctas;
    num_kb = kbs;
    next_tile = SHARED ? tiles : cta;
    stride = ctas;
    total_tiles = tiles;
  }
  __device__ __forceinline__ bool next(Segment& sg) {
    if (SHARED) {
      if (u >= end) return false;
      sg.tile = (int)(u / num_kb);
      sg.kb0 = (int)(u - (long long)sg.tile * num_kb);
      const long long left = end - u;
      const int room = num_kb - sg.kb0;
      sg.kb1 = sg.kb0 + (int)(left < room ? left : room);
      u += sg.kb1 - sg.kb0;
      return true;
    }
    if (next_tile >= total_tiles) return false;
    sg.tile = next_tile;
    sg.kb0 = 0;
    sg.kb1 = num_kb;
    next_tile += stride;
    return true;
  }
};

#define SK_SLOT_FLOATS (BM * 256)                    // a CTA's slot in the workspace: one 128 x 256 accumulator
// where a CTA leaves the sums of a tile it only did part of (one slot per CTA), and the words that say they are there
__device__ float* d_split_ws = nullptr;
__device__ int* d_split_flags = nullptr;

template <int BN, int STAGES, typename TC, bool SWIGLU, bool ROPE = false, bool SHARED = false>
__global__ void __launch_bounds__(192) gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                 const __grid_constant__ CUtensorMap map_w,
                                                                 const GemmArgs args, const RopeArgs rope) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN;                  // 256 or 512: a power of two
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(tiles + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;               // [2]
  uint64_t* acc_empty = acc_full + 2;                // [2]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;   // known to be uniform
  const int M = args.rows_wide, N = args.rows_narrow;
  const int bn = args.bn;                            // columns of a tile: at most BN, the ring's room
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + bn - 1) / bn;
  const int total_tiles = tiles_m * tiles_n;
  const int num_kb = (args.K + BK - 1) / BK;
  const int ctas = (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  if (warp == 0) {
    {
      // (the whole warp walks the loop and waits, an elected lane requests: see the MMA warp)
      const bool leader = elect_one();
      // Arms stage s and requests the bn weight rows from n0 for k block kb: one tensor tile, or,
      // from a packed matrix, the rows' share of each 16 KB tile they lie in (eight rows are 1 KB
      // of a tile, so rows from a multiple of 16 are a contiguous piece that lands on a swizzle
      // boundary; rows past the last tile are left out: their columns are never stored).
      const int w_rows = ((N + BM - 1) / BM) * BM;
      auto load_w = [&](int s, int kb, int n0) {
        uint8_t* dst = tiles + s * STAGE_BYTES + A_BYTES;
        if (!leader) return;
        if (args.packed) {
          const int end = n0 + bn < w_rows ? n0 + bn : w_rows;
          mbar_expect_tx(&full[s], A_BYTES + (end - n0) * (BK * 2));
          for (int row = n0; row < end;) {
            const int t = row / BM, r0 = row % BM;
            const int n = (end - t * BM < BM ? end - t * BM : BM) - r0;
            bulk_load_1d(dst + (row - n0) * (BK * 2), args.packed + ((size_t)t * num_kb + kb) * (size_t)A_BYTES + r0 * (BK * 2),
                         &full[s], n * (BK * 2));
            row += n;
          }
        } else {
          mbar_expect_tx(&full[s], A_BYTES + bn * (BK * 2));
          tma_load_2d(dst, &map_w, &full[s], kb * BK, n0);
        }
      };
      // the first stages' weight tiles do not depend on the kernel ahead
      int it = 0;
      bool first = true, ok = true;
      Share<SHARED> sh(blockIdx.x, ctas, total_tiles, num_kb);
      Segment sg;
      while (ok && sh.next(sg)) {
        const int m0 = (sg.tile % tiles_m) * BM, n0 = (sg.tile / tiles_m) * bn;
        int kb = sg.kb0;
        if (first) {
          const int len = sg.kb1 - sg.kb0;
          const int pre = len < STAGES ? len : STAGES;
          for (int k = 0; k < pre; ++k) load_w(k, sg.kb0 + k, n0);
          pdl_wait();
          if (leader)
            for (int k = 0; k < pre; ++k) tma_load_2d(tiles + k * STAGE_BYTES, &map_x, &full[k], (sg.kb0 + k) * BK, m0);
          __syncwarp();
          kb = sg.kb0 + pre;
          it = pre;
          first = false;
        }
        for (; kb < sg.kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, args.err, 1)) { ok = false; break; }
          load_w(s, kb, n0);
          if (leader) tma_load_2d(tiles + s * STAGE_BYTES, &map_x, &full[s], kb * BK, m0);
          __syncwarp();
        }
      }
      if (first) pdl_wait();
    }
  } else if (warp == 1) {
    {
      // The whole warp walks the loop and waits; one elected lane issues.  (Under a branch on the lane number
      // the products' operands are per-thread values, moved one at a time to the uniform registers the
      // instruction wants: some 85 clocks a product, more than a product 128 columns wide takes.)
      const bool leader = elect_one();
      const uint32_t idesc = umma_idesc(BM, bn);
      int it = 0, local = 0;
      bool ok = true;
      Share<SHARED> sh(blockIdx.x, ctas, total_tiles, num_kb);
      Segment sg;
      while (ok && sh.next(sg)) {
        const int b = local & 1;
        // the epilogue must have drained this accumulator (two pieces of work ago)
        ok = mbar_wait(&acc_empty[b], ((local >> 1) & 1) ^ 1, args.err, 4);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * BN);
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(&full[s], ph, args.err, 2);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES);
          const uint64_t da = umma_desc(a_addr), db = umma_desc(a_addr + A_BYTES);
          if (leader) {
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
              umma_f16(d_tmem, da + 2 * kk, db + 2 * kk, idesc, (kb > sg.kb0 || kk > 0) ? 1u : 0u);
            umma_commit(&empty[s]);
          }
          __syncwarp();
        }
        if (leader) umma_commit(&acc_full[b]);
        __syncwarp();
        ++local;
      }
    }
  } else {
    pdl_wait();                                      // C (and the workspace) may still be in use by the kernel ahead
    const int q = warp & 3;
    TC* C = (TC*)args.C;
    int local = 0;
    const long long units = (long long)total_tiles * num_kb;       // shared: all tiles are
    float* const sk_ws = SHARED ? d_split_ws : nullptr;
    int* const sk_flags = SHARED ? d_split_flags : nullptr;
    Share<SHARED> sh(blockIdx.x, ctas, total_tiles, num_kb);
    Segment sg;
    while (sh.next(sg)) {
      const int b = local & 1;
      const int m0 = (sg.tile % tiles_m) * BM, n0 = (sg.tile / tiles_m) * bn;
      // every thread polls: the arrivals below need all 128 of them, timed out or not
      bool ok = mbar_wait(&acc_full[b], (local >> 1) & 1, args.err, 3);
      tc_fence_after();
      const int row_in_tile = q * 32 + lane;
      const int row = m0 + row_in_tile;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * BN);
      if (SHARED && ok && sg.kb0 > 0) {
        // only later k blocks of the tile are this CTA's: its sums go to its slot, for the tile's owner
        // (as [32-column chunk][float4 of the chunk][row], so that a warp's stores and the owner's loads are contiguous)
        float4* slot = (float4*)(sk_ws + (size_t)blockIdx.x * SK_SLOT_FLOATS) + row_in_tile;
#pragma unroll 1
        for (int c0 = 0; c0 < bn; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + c0, r);
          tmem_wait_ld();
          float4* dst = slot + (size_t)(c0 >> 5) * 8 * BM;
#pragma unroll
          for (int v = 0; v < 8; ++v)
            dst[v * BM] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
        }
        __threadfence();                             // the sums before the flag
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (q == 0 && lane == 0) atomicExch(sk_flags + blockIdx.x, 1);
      } else if (ok) {
        if (SHARED && sg.kb1 < num_kb) {
          // The tile's later k blocks are the following CTAs' (every CTA has some: the host shares tiles only
          // then).  They did that work first of all, while this CTA did its own part, so the wait for
          // their flags is short; it is bounded like every other.  Their sums are added to this
          // accumulator in tensor memory, chunk by chunk and in CTA order, before the epilogue reads it.
          int n = 0;
          for (long long at = units * (blockIdx.x + 1) / ctas; at < (long long)(sg.tile + 1) * num_kb; at = units * (blockIdx.x + 1 + n) / ctas) ++n;
          for (int j = 0; j < n; ++j) {
            volatile int* flag = sk_flags + blockIdx.x + 1 + j;
            uint32_t spins = 0;
            while (*flag == 0 && ++spins < WAIT_LIMIT) {}
            if (*flag == 0) ok = false;
          }
          {  // all 128 threads go on, or none: one that gave up takes the others with it
            uint32_t seen = ok, all_seen;
            asm volatile("{ .reg .pred p, q; setp.ne.u32 p, %1, 0; bar.red.and.pred q, 1, 128, p; selp.u32 %0, 1, 0, q; }"
                         : "=r"(all_seen) : "r"(seen) : "memory");
            ok = all_seen != 0;
            if (!ok && q == 0 && lane == 0) atomicExch(args.err, 7);
          }
          if (ok) {
            __threadfence();                         // the flags before the sums
            const float4* first = (const float4*)(sk_ws + (size_t)(blockIdx.x + 1) * SK_SLOT_FLOATS) + row_in_tile;
            const int items = ((bn + 31) >> 5) * n;  // (chunk, contributor) pairs, contributors fastest
            // two pairs' loads are in flight while a third is added: the trip to L2 is what this loop waits for
            auto issue = [&](int i, float4* p) {
              const int ch = i / n, j = i - ch * n;
              const float4* src = first + (size_t)j * (SK_SLOT_FLOATS / 4) + (size_t)ch * 8 * BM;
#pragma unroll
              for (int v = 0; v < 8; ++v) p[v] = __ldcg(src + v * BM);
            };
            uint32_t r[32];
            auto consume = [&](int i, const float4* p) {
              const int ch = i / n, j = i - ch * n;
              if (j == 0) { tmem_ld32(taddr + ch * 32, r); tmem_wait_ld(); }
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                r[4 * v] = __float_as_uint(__uint_as_float(r[4 * v]) + p[v].x);
                r[4 * v + 1] = __float_as_uint(__uint_as_float(r[4 * v + 1]) + p[v].y);
                r[4 * v + 2] = __float_as_uint(__uint_as_float(r[4 * v + 2]) + p[v].z);
                r[4 * v + 3] = __float_as_uint(__uint_as_float(r[4 * v + 3]) + p[v].w);
              }
              if (j == n - 1) tmem_st32(taddr + ch * 32, r);
            };
            float4 pa[8], pb[8], pc[8];
            issue(0, pa);
            if (1 < items) issue(1, pb);
#pragma unroll 1
            for (int i = 0; i < items; i += 3) {
              if (i + 2 < items) issue(i + 2, pc);
              consume(i, pa);
              if (i + 3 < items) issue(i + 3, pa);
              if (i + 1 < items) consume(i + 1, pb);
              if (i + 4 < items) issue(i + 4, pb);
              if (i + 2 < items) consume(i + 2, pc);
            }
            tmem_wait_st();
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");      // every thread has read the slots: their flags go down for the next launch
          if (q == 0 && lane == 0)
            for (int j = 0; j < n; ++j) atomicExch(sk_flags + blockIdx.x + 1 + j, 0);
        }
        if (ok && ROPE) {
          if (rope.hd == 128) rope_store_row<128>(rope, (bf16*)args.C, args.ldc, taddr, row, row < M, n0, bn, N);
          else rope_store_row<64>(rope, (bf16*)args.C, args.ldc, taddr, row, row < M, n0, bn, N);
        } else if (ok) {
#pragma unroll 1
          for (int c0 = 0; c0 < bn; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(taddr + c0, r);                  // a last chunk of 16 columns reads on into unused ones
            tmem_wait_ld();
            if (row >= M || n0 + c0 >= N) continue;
            store_chunk<TC, SWIGLU>(C, args.ldc, row, n0 + c0, (N - (n0 + c0)) < (bn - c0) ? (N - (n0 + c0)) : (bn - c0), r);
          }
        }
      }
      tc_fence_before();
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[b])) : "memory");
      if (!ok) break;
      ++local;
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------- host side
// Streaming multiprocessors of the current device, asked once.
int device_sms() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

template <int BN, int STAGES, typename TC, bool SWIGLU = false>
int launch(const CUtensorMap& mw, const CUtensorMap& mn, const GemmArgs& args, dim3 grid, cudaStream_t st,
           const NormArgs& norm = NormArgs()) {
  constexpr int smem = STAGES * (BM * BK * 2 + BN * BK * 2) + 1024 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, TC, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  // split-K CTAs of a tile (grid.z of them) are one cluster
  return qv_launch_cluster(gemm_tc_kernel<BN, STAGES, TC, SWIGLU>, grid, dim3(192), (size_t)smem, st, dim3(1, 1, grid.z), mw, mn, args, norm);
}

float* g_split_ws = nullptr;             // see qv_gemm_bf16_set_split_workspace
int* g_split_flags = nullptr;
int g_split_ctas = 0;

// Are the tiles of a product shared between the CTAs?  Where they fill at most three quarters of the
// SMs, each tile is cut into no more than eight pieces, the tiles have 128 columns and a tile's walk along
// K is long enough (4,096 or more): handing over and adding the partial sums costs ~10 us.  Measured, whole
// against shared: 4096 x 14336 at 128 tokens 72 -> 36 us, at 384 tokens 76 -> 64 us; 4096 x 4096 at 128 tokens
// 23.9 -> 21.6 us, at 384 tokens no change; 2048 x 2048 at 256 tokens (K too short) 14.3 -> 18.4 us; tiles of 256
// columns, whose partial sums are twice as large, 5120 x 13824 at 512 tokens 90 -> 98 us.
bool share_tiles(int total_tiles, int num_kb, int bn) {
  const int sms = device_sms();
  return g_split_ws != nullptr && g_split_ctas >= sms && bn <= 128 && total_tiles * 4 <= sms * 3 && total_tiles * 8 >= sms && num_kb >= 64;
}

template <int BN, int STAGES, typename TC, bool SWIGLU, bool ROPE, bool SHARED>
int launch_persistent_kernel(const CUtensorMap& mx, const CUtensorMap& mw, const GemmArgs& args, int ctas, cudaStream_t st, const RopeArgs& rope) {
  constexpr int smem = STAGES * (BM * BK * 2 + BN * BK * 2) + 1024 + 256;
  static bool configured = false;
  auto kernel = gemm_tc_persistent_kernel<BN, STAGES, TC, SWIGLU, ROPE, SHARED>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return qv_launch(kernel, dim3(ctas), dim3(192), (size_t)smem, st, mx, mw, args, rope);
}

template <int BN, int STAGES, typename TC, bool SWIGLU, bool ROPE = false>
int launch_persistent(const CUtensorMap& mx, const CUtensorMap& mw, const GemmArgs& args, int total_tiles, cudaStream_t st,
                      const RopeArgs& rope = RopeArgs()) {
  const int sms = device_sms();
  // tiles are shared only by products with the plain epilogue (the narrow, long ones are output and down projections)
  if (!SWIGLU && !ROPE && share_tiles(total_tiles, (args.K + BK - 1) / BK, args.bn)) {
    return launch_persistent_kernel<BN, STAGES, TC, false, false, true>(mx, mw, args, sms, st, rope);
  }
  return launch_persistent_kernel<BN, STAGES, TC, SWIGLU, ROPE, false>(mx, mw, args, total_tiles < sms ? total_tiles : sms, st, rope);
}

}  // namespace

// The workspace through which CTAs of the persistent kernel hand partial sums of a shared tile to its
// owner: `ctas` slots of 128 x 256 floats and `ctas` flag words that are zero (the kernel leaves them
// zero).  It belongs to the caller, is used by every later product of many tokens that shares tiles and
// must outlive them; such products must not run at the same time on different streams.  Null: tiles are
// never shared.
extern "C" void qv_gemm_bf16_set_split_workspace(float* slots, int* flags, int ctas) {
  g_split_ws = slots;
  g_split_flags = flags;
  g_split_ctas = slots && flags ? ctas : 0;
  // the kernels read the addresses from device words (set here, once; not on the launch path)
  if (cudaMemcpyToSymbol(d_split_ws, &slots, sizeof(slots)) != cudaSuccess || cudaMemcpyToSymbol(d_split_flags, &flags, sizeof(flags)) != cudaSuccess)
    g_split_ctas = 0;
}
extern "C" long long qv_gemm_bf16_split_slot_bytes() { return (long long)SK_SLOT_FLOATS * 4; }

// Columns of the persistent kernel's tiles: 0 (default) chooses per product, else the given width
// (a multiple of 16, of 32 with the fused activation, at most 256; for comparison and tests).
static int g_prefill_bn = 0;
extern "C" void qv_gemm_bf16_set_prefill_bn(int v) { g_prefill_bn = v; }

// The tile width of a product.  A k block of a 128 x bn tile costs a fixed part worth about 500
// columns beside its bn columns (measured: the shared-memory fill, not the MMA, sets the pace), so
// the widest tile wins unless half-width tiles still fit in one wave of CTAs, which then finishes
// sooner (4096 x 14336 at 512 tokens: 76.9 us at 128 columns, 88.1 us at 256).
static int choose_tile_width(int tiles_m, int N, int K, int step) {
  (void)step;
  (void)K;
  return tiles_m * ((N + 127) / 128) <= device_sms() ? 128 : 256;
}

// K splits of the few-token kernel and the k blocks of each.
// `tokens`: the rows of the narrow side; `least`: the fewest splits the epilogue works with.
static int swap_splits(int tiles, int total_kb, int epilogue, int force_splits, int tokens, int least, int* per_split) {
  int splits = 1;
  if (epilogue == 1) splits = 1;                  // the fused activation needs whole sums
  else if (force_splits > 0) splits = force_splits;
  else if (tiles < (2 * device_sms()) / 3) {      // too few CTAs to pull full bandwidth: split along K
    // a power of two, at most 4: clusters of 8 CTAs do not all find room at once (measured: a
    // 2048 x 8192 product takes 22.5 us at 8 splits, 13.2 us at 4), and at most 4/3 CTAs per SM in all
    while (splits < 4 && tiles * splits * 2 <= device_sms() + device_sms() / 3 && total_kb / (splits * 2) >= 4) splits *= 2;
    // From 32 tokens on the partial sums that cross between the CTAs of a cluster weigh more than the SMs a
    // second, partly filled round of CTAs adds (6144 x 4096, 48 tiles: 64 tokens 18.2 us at 4 splits, 16.3 at 2,
    // 14.6 at 1; 32 tokens 14.1 / 13.6 / 13.4; 8 tokens 11.3 / 11.8 / 12.6)
    if (tokens >= 32 && tiles * splits > device_sms()) splits = least;
  }
  if (splits > total_kb) splits = total_kb;
  const int per = (total_kb + splits - 1) / splits;
  *per_split = per;
  return (total_kb + per - 1) / per;              // no empty split
}

// C (bf16 or f32) [M,N] = A (bf16) [M,K] * W (bf16) [N,K]^T.  Returns QV_ERR_UNSUPPORTED for shapes
// the tensor-core path does not take (the caller then uses the CUDA-core kernel):
// K not a multiple of 8 elements, or operands whose rows do not start on 16-byte boundaries.
static int gemm_bf16_entry(void* C, const void* A, const void* W, const void* packed, int M, int N, int K, int lda, int ldw, int ldc,
                           int c_dt, int* err, int force_splits, int epilogue, void* stream) {
  // epilogue 0: C[M,N] = A W^T.  epilogue 1: W's rows are 16 gate rows / 16 up rows interleaved and
  // C[M,N/2] = silu(gate) * up (bfloat16 out, N a multiple of 32).
  if (M <= 0 || N <= 0) return 0;
  if (epilogue != 0 && (epilogue != 1 || c_dt != QV_DT_BF16 || (N & 31))) return QV_ERR_UNSUPPORTED;
  if (K < 8 || (K & 7) || (lda & 7) || (ldw & 7)) return QV_ERR_UNSUPPORTED;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)packed & 15)) return QV_ERR_UNSUPPORTED;
  if (c_dt != QV_DT_BF16 && c_dt != QV_DT_F32) return QV_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  GemmArgs args;
  args.C = C; args.err = err; args.packed = nullptr; args.bn = 0;
  args.K = K; args.ldc = ldc;
  const int total_kb = (K + BK - 1) / BK;
  CUtensorMap mw, mn;
  if (M <= 64) {
    // swap: weights on the 128-row side, tokens on the narrow side
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    const int tiles = (N + BM - 1) / BM;
    int per = 0;
    const int splits = swap_splits(tiles, total_kb, epilogue, force_splits, M, 1, &per);
    args.rows_wide = N; args.rows_narrow = M; args.kblocks_per_split = per; args.splits = splits;
    if (!make_map(&mn, A, M, K, lda, bn)) return QV_ERR_UNSUPPORTED;
    if (packed) { args.packed = (const uint8_t*)packed; mw = mn; }
    else if (!W || !make_map(&mw, W, N, K, ldw, BM)) return QV_ERR_UNSUPPORTED;
    dim3 grid(tiles, 1, splits);
#define SWAP_LAUNCH(BN_, ST_)                                                                     \
  (c_dt == QV_DT_BF16 ? launch<BN_, ST_, bf16>(mw, mn, args, grid, st) : launch<BN_, ST_, float>(mw, mn, args, grid, st))
    if (epilogue == 1) {
      if (bn == 16) return launch<16, 6, bf16, true>(mw, mn, args, grid, st);
      if (bn == 32) return launch<32, 5, bf16, true>(mw, mn, args, grid, st);
      return launch<64, 4, bf16, true>(mw, mn, args, grid, st);
    }
    const bool one_wave = tiles * splits <= device_sms();     // every CTA resident at once, one per SM: deeper rings
    if (bn == 16) return one_wave ? SWAP_LAUNCH(16, 12) : SWAP_LAUNCH(16, 6);
    if (bn == 32) return one_wave ? SWAP_LAUNCH(32, 10) : SWAP_LAUNCH(32, 5);
    return one_wave ? SWAP_LAUNCH(64, 8) : SWAP_LAUNCH(64, 4);
#undef SWAP_LAUNCH
  }
  // many tokens: tokens on the 128-row side, 128 weight rows per tile
  if (!W && !packed) return QV_ERR_UNSUPPORTED;
  args.packed = (const uint8_t*)packed;
  args.rows_wide = M; args.rows_narrow = N; args.kblocks_per_split = total_kb; args.splits = 1;
  const int step = epilogue == 1 ? 32 : 16;
  const int bn = g_prefill_bn > 0 ? g_prefill_bn : choose_tile_width((M + BM - 1) / BM, N, K, step);
  // persistent kernel, 128 x bn tiles, accumulator double-buffered in tensor memory
  if (bn < step || bn > 256 || bn % step) return QV_ERR_UNSUPPORTED;
  args.bn = bn;
  if (!make_map(&mw, A, M, K, lda, BM)) return QV_ERR_UNSUPPORTED;
  if (packed) mn = mw;
  else if (!make_map(&mn, W, N, K, ldw, bn)) return QV_ERR_UNSUPPORTED;
  const int total_tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
  if (epilogue == 1) return launch_persistent<256, 4, bf16, true>(mw, mn, args, total_tiles, st);
  if (c_dt == QV_DT_BF16) return launch_persistent<256, 4, bf16, false>(mw, mn, args, total_tiles, st);
  return launch_persistent<256, 4, float, false>(mw, mn, args, total_tiles, st);
}

// The QKV projection of more than 64 tokens with the rotation of query and key heads and the write
// of keys and values into the paged cache done in the product's epilogue (from the float32
// accumulators; the separate pass over the product's output is saved: 28.4 against 29.4 ms for a
// 2,048-token prompt at Llama-3.1-8B sizes).  The same fusion in the few-token kernel, whose
// epilogue is on every decode step's critical path, measured 0.7 % slower than the separate
// rotary kernel and is not built.  C [M, (H + 2 Hkv) hd] gets
// the rotated query heads; its key and value columns are left unwritten.  Head sizes 64 and 128 with
// all dims rotated; QV_ERR_UNSUPPORTED otherwise (the caller then runs the product and the rotation
// as two kernels).
extern "C" int qv_gemm_bf16_qkv_rope(void* C, const void* A, const void* packed, int M, int K, int lda, int ldc, int* err,
                                     const float* cos_sin, int table_rows, const int* tok_pos, const int* tok_seg,
                                     const int* block_table, int max_blocks, void* cache, int H, int Hkv, int hd, int page_size,
                                     void* stream) {
  if (M <= 64 || !packed || !cache || !cos_sin) return QV_ERR_UNSUPPORTED;
  if ((hd != 64 && hd != 128) || H <= 0 || Hkv <= 0 || page_size <= 0 || table_rows <= 0) return QV_ERR_UNSUPPORTED;
  const long long n_ll = (long long)(H + 2 * Hkv) * hd;
  if (n_ll > 0x7fffffffLL) return QV_ERR_TOO_LARGE;
  const int N = (int)n_ll;
  if (K < 8 || (K & 7) || (lda & 7) || (ldc & 7) || ldc < N) return QV_ERR_UNSUPPORTED;
  if (((uintptr_t)A & 15) || ((uintptr_t)C & 15) || ((uintptr_t)packed & 15) || ((uintptr_t)cache & 15) || ((uintptr_t)cos_sin & 15))
    return QV_ERR_UNSUPPORTED;
  GemmArgs args;
  args.C = C; args.err = err; args.packed = (const uint8_t*)packed;
  args.K = K; args.ldc = ldc;
  RopeArgs ra;
  ra.cos_sin = (const float2*)cos_sin; ra.tok_pos = tok_pos; ra.tok_seg = tok_seg; ra.block_table = block_table;
  ra.cache = (bf16*)cache; ra.table_rows = table_rows; ra.max_blocks = max_blocks;
  ra.H = H; ra.Hkv = Hkv; ra.hd = hd; ra.page_size = page_size;
  args.rows_wide = M; args.rows_narrow = N; args.kblocks_per_split = (K + BK - 1) / BK; args.splits = 1;
  args.bn = g_prefill_bn > 0 ? g_prefill_bn : choose_tile_width((M + BM - 1) / BM, N, K, 16);
  if (args.bn > 256 || args.bn % hd) return QV_ERR_UNSUPPORTED;      // whole heads per tile
  CUtensorMap mx;
  if (!make_map(&mx, A, M, K, lda, BM)) return QV_ERR_UNSUPPORTED;
  const int total_tiles = ((M + BM - 1) / BM) * ((N + args.bn - 1) / args.bn);
  return launch_persistent<256, 4, bf16, false, true>(mx, mx, args, total_tiles, (cudaStream_t)stream, ra);
}

// A product of up to 64 tokens with the neighbouring RMS norm folded in (see NormArgs).  With
// `residual`: C [M,N] (bfloat16) = (residual += A W^T) * norm_w and ssq_out [ceil(N/128)][64] gets the
// sums of squares; the product must be one that is split along K (its first CTA holds whole sums).
// With `ssq_in` (tiles_in x 64, of a stream of 1/inv_d features): every token's sums are scaled by
// rsqrt(mean of squares + eps) before they are stored (or, epilogue 1, before SwiGLU).
// QV_ERR_UNSUPPORTED, with nothing written, for anything else.
extern "C" int qv_gemm_bf16_norm(void* C, const void* A, const void* packed, int M, int N, int K, int lda, int ldc, int c_dt,
                                 int* err, int epilogue, float* residual, int ld_res, const float* norm_w, float* ssq_out,
                                 const float* ssq_in, int tiles_in, float inv_d, float eps, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || !packed || (epilogue != 0 && epilogue != 1)) return QV_ERR_UNSUPPORTED;
  if (epilogue == 1 && (c_dt != QV_DT_BF16 || (N & 31))) return QV_ERR_UNSUPPORTED;
  if (c_dt != QV_DT_BF16 && c_dt != QV_DT_F32) return QV_ERR_UNSUPPORTED;
  if (K < 8 || (K & 7) || (lda & 7)) return QV_ERR_UNSUPPORTED;
  if (((uintptr_t)A & 15) || ((uintptr_t)packed & 15)) return QV_ERR_UNSUPPORTED;
  if (residual && (!norm_w || !ssq_out || epilogue != 0 || c_dt != QV_DT_BF16 || ld_res < N)) return QV_ERR_UNSUPPORTED;
  if (ssq_in && (tiles_in <= 0 || !(inv_d > 0.f))) return QV_ERR_UNSUPPORTED;
  const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  const int tiles = (N + BM - 1) / BM, total_kb = (K + BK - 1) / BK;
  int per = 0;
  const int splits = swap_splits(tiles, total_kb, epilogue, 0, M, residual ? 2 : 1, &per);
  if (residual && splits < 2) return QV_ERR_UNSUPPORTED;
  GemmArgs args;
  args.C = C; args.err = err; args.packed = (const uint8_t*)packed; args.bn = 0;
  args.K = K; args.ldc = ldc;
  args.rows_wide = N; args.rows_narrow = M; args.kblocks_per_split = per; args.splits = splits;
  NormArgs na;
  na.residual = residual; na.norm_w = norm_w; na.ssq_out = ssq_out; na.ssq_in = ssq_in;
  na.ld_res = ld_res; na.tiles_in = tiles_in; na.inv_d = inv_d; na.eps = eps;
  CUtensorMap mn;
  if (!make_map(&mn, A, M, K, lda, bn)) return QV_ERR_UNSUPPORTED;
  dim3 grid(tiles, 1, splits);
  cudaStream_t st = (cudaStream_t)stream;
#define NORM_LAUNCH(BN_, ST_)                                                                     \
  (c_dt == QV_DT_BF16 ? launch<BN_, ST_, bf16>(mn, mn, args, grid, st, na) : launch<BN_, ST_, float>(mn, mn, args, grid, st, na))
  if (epilogue == 1) {
    if (bn == 16) return launch<16, 6, bf16, true>(mn, mn, args, grid, st, na);
    if (bn == 32) return launch<32, 5, bf16, true>(mn, mn, args, grid, st, na);
    return launch<64, 4, bf16, true>(mn, mn, args, grid, st, na);
  }
  const bool one_wave = tiles * splits <= device_sms();
  if (bn == 16) return one_wave ? NORM_LAUNCH(16, 12) : NORM_LAUNCH(16, 6);
  if (bn == 32) return one_wave ? NORM_LAUNCH(32, 10) : NORM_LAUNCH(32, 5);
  return one_wave ? NORM_LAUNCH(64, 8) : NORM_LAUNCH(64, 4);
#undef NORM_LAUNCH
}

extern "C" int qv_gemm_bf16_tc(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc,
                               int c_dt, int* err, int force_splits, int epilogue, void* stream) {
  return gemm_bf16_entry(C, A, W, nullptr, M, N, K, lda, ldw, ldc, c_dt, err, force_splits, epilogue, stream);
}

// As qv_gemm_bf16_tc, with the weight matrix given as packed tiles (qv_pack_weight_tiles): every CTA
// then fetches its weight tiles with contiguous 16 KB copies, which an SM takes in ~1.6x faster than
// tensor tiles of 128-byte rows and HBM serves ~15 % faster.
extern "C" int qv_gemm_bf16_packed(void* C, const void* A, const void* packed, int M, int N, int K, int lda, int ldc, int c_dt,
                                   int* err, int force_splits, int epilogue, void* stream) {
  if (!packed) return QV_ERR_UNSUPPORTED;
  return gemm_bf16_entry(C, A, nullptr, packed, M, N, K, lda, K, ldc, c_dt, err, force_splits, epilogue, stream);
}

// ---------------------------------------------------------------- packed weights
// W [N, K] (row stride ldw) -> tiles of 128 rows x 64 k, tile (t, kb) at byte ((t * kblocks + kb) * 16384),
// each stored as the shared-memory image the MMA reads (128-byte rows, 16-byte chunk c of row r at
// chunk c ^ (r % 8)), zero where the matrix ends.
__global__ void pack_weight_tiles_kernel(uint4* __restrict__ out, const bf16* __restrict__ W, int N, int K, int ldw, int kblocks) {
  const int kb = blockIdx.x, t = blockIdx.y;
  const int r = threadIdx.x >> 3, c = threadIdx.x & 7;      // 16 rows x 8 chunks per pass
  uint4* tile = out + ((size_t)t * kblocks + kb) * (A_TILE_BYTES / 16);
  for (int rr = r; rr < BM; rr += 16) {
    const int row = t * BM + rr, k0 = kb * BK + c * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < N && k0 < K) v = *(const uint4*)(W + (size_t)row * ldw + k0);
    tile[(rr >> 3) * 64 + (rr & 7) * 8 + (c ^ (rr & 7))] = v;
  }
}

extern "C" long long qv_packed_weight_bytes(int N, int K) {
  return (long long)((N + BM - 1) / BM) * ((K + BK - 1) / BK) * A_TILE_BYTES;
}

extern "C" int qv_pack_weight_tiles(void* out, const void* W, int N, int K, int ldw, void* stream) {
  if (N <= 0 || K < 8 || (K & 7) || (ldw & 7) || ((uintptr_t)W & 15) || ((uintptr_t)out & 15)) return QV_ERR_UNSUPPORTED;
  const int tiles = (N + BM - 1) / BM, kblocks = (K + BK - 1) / BK;
  if (tiles > 65535) return QV_ERR_TOO_LARGE;
  pack_weight_tiles_kernel<<<dim3(kblocks, tiles), 128, 0, (cudaStream_t)stream>>>((uint4*)out, (const bf16*)W, N, K, ldw, kblocks);
  return (int)cudaGetLastError();
}
