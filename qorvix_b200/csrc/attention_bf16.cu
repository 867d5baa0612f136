// Causal grouped-query attention over the paged bfloat16 cache on the tensor cores, for
// serving: a flash-attention kernel for prompt portions and a split-KV kernel for decoded
// tokens.  Formula and masking are those of the reference's CPU model
// (runtime/src/text_model.cpp:83-114: kv head = h / (H/Hkv), score = q.k / sqrt(hd) for keys up
// to the query's position, softmax, weighted sum of V); its CUDA kernel keeps every score of a
// sequence in shared memory and runs the softmax on one thread
// (cuda/src/cuda_backend.cu:347-395), which neither scales to long contexts nor batches.
//
// Both kernels work on blocks of 16 keys with mma.sync m16n8k16 (bf16 in, float32 out) and an
// online softmax in float32.  Operands go from global memory (L1/L2) straight into MMA
// fragments, without shared memory: a dot product may sum its terms in any order, so the k
// index of a fragment is mapped to head dims in the order in which one 16-byte load delivers
// them (the same mapping for Q and K), and for P.V the output dims are permuted likewise, with
// byte permutes pairing the values of two keys.  Keys are read through the request's block
// table; a block of 16 keys never straddles a page (pages are multiples of 16 tokens).
//
//   prefill: one CTA = 64 query tokens of one head (4 warps x 16 rows); each warp walks the
//            keys of its rows.  Grid (query tiles, heads, segments).
//   decode:  one CTA = one token, one kv head, one slice of the keys; the rows of the MMA
//            tile are the query heads that share the kv head; the 4 warps take alternate
//            16-key blocks and merge through shared memory; slices merge in a second kernel.
#include "attention_mma.cuh"
#include "tc_common.cuh"

namespace {

// ---------------------------------------------------------------- prefill
template <int HD>
__global__ void __launch_bounds__(128) attn_prefill_kernel(bf16* __restrict__ out, int ld_out, const bf16* __restrict__ q, int ld_q,
                                                           const bf16* __restrict__ cache, const int* __restrict__ seg_q_start,
                                                           const int* __restrict__ seg_pos0, const int* __restrict__ block_table,
                                                           int max_blocks, int H, int Hkv, int page, int window, float scale_log2) {
  pdl_wait();
  pdl_launch_dependents();
  // grid (heads, query tiles, segments), the last query tile (most keys) first: CTAs are handed out
  // x-fastest, so the longest work starts first
  const int seg = blockIdx.z, h = blockIdx.x;
  const int q0 = seg_q_start[seg], qlen = seg_q_start[seg + 1] - q0;
  const int tile0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * 64;
  if (tile0 >= qlen) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const int r0 = tile0 + warp * 16;                 // first row of this warp within the segment
  if (r0 >= qlen) return;
  const int pos0 = seg_pos0[seg];
  const int kvh = h / (H / Hkv);
  const int* bt = block_table + (size_t)seg * max_blocks;
  const int rows[2] = {r0 + g, r0 + g + 8};
  const bool valid[2] = {rows[0] < qlen, rows[1] < qlen};
  QFrag<HD> qf;
  load_q<HD>(qf, valid[0] ? q + (size_t)(q0 + rows[0]) * ld_q + (size_t)h * HD : nullptr,
             valid[1] ? q + (size_t)(q0 + rows[1]) * ld_q + (size_t)h * HD : nullptr, tg);
  int lo[2], hi[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    hi[r] = valid[r] ? pos0 + rows[r] : -1;
    lo[r] = (window > 0 && hi[r] - window + 1 > 0) ? hi[r] - window + 1 : 0;
  }
  const int last_row = (r0 + 15 < qlen ? r0 + 15 : qlen - 1);
  const int k_end = pos0 + last_row;                              // last key any row of this warp sees
  int k_begin = 0;
  if (window > 0) { const int f = pos0 + r0 - window + 1; k_begin = f > 0 ? (f & ~15) : 0; }
  RowState<HD> st;
  st.init();
  const size_t page_elems = (size_t)2 * Hkv * page * HD;
  const size_t v_off = (size_t)Hkv * page * HD;
  for (int base = k_begin; base <= k_end; base += 16) {
    const bf16* kblk = cache + (size_t)bt[base / page] * page_elems + ((size_t)kvh * page + (base % page)) * HD;
    block16<HD, false>(st, qf, kblk, kblk + v_off, base, lo, hi, scale_log2, g, tg);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
    st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (!valid[r]) continue;
    const float inv = 1.f / st.l[r];
    bf16* orow = out + (size_t)(q0 + rows[r]) * ld_out + (size_t)h * HD;
#pragma unroll
    for (int i = 0; i < Shape<HD>::NT; ++i) {
      orow[out_dim<HD>(i, 2 * tg)] = __float2bfloat16_rn(st.o[i][2 * r] * inv);
      orow[out_dim<HD>(i, 2 * tg + 1)] = __float2bfloat16_rn(st.o[i][2 * r + 1] * inv);
    }
  }
}

// ---------------------------------------------------------------- prefill, shared-memory tiles
// For head sizes 64 and 128: 64 query rows and 64-key tiles of K and V staged in shared memory
// with cp.async (two stages, XOR-swizzled 16-byte chunks), shared by the CTA's four warps and
// read with ldmatrix (transposed for V).  Same arithmetic as the register-direct kernel above;
// it moves each key and value once per 64 queries instead of once per 16.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t* r, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t* r, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

template <int HD>
__global__ void __launch_bounds__(128) attn_prefill_tile_kernel(bf16* __restrict__ out, int ld_out, const bf16* __restrict__ q, int ld_q,
                                                                const bf16* __restrict__ cache, const int* __restrict__ seg_q_start,
                                                                const int* __restrict__ seg_pos0, const int* __restrict__ block_table,
                                                                int max_blocks, int H, int Hkv, int page, int window, float scale_log2) {
  extern __shared__ __align__(128) uint8_t smem_bytes[];
  constexpr int CH = HD / 8;                        // 16-byte chunks per row
  constexpr int KS = HD / 16;                       // k steps of a dot product over the head
  bf16* sQ = (bf16*)smem_bytes;                     // [64][HD]
  bf16* sK = sQ + 64 * HD;                          // [2][64][HD]
  bf16* sV = sK + 2 * 64 * HD;                      // [2][64][HD]
  pdl_wait();
  pdl_launch_dependents();
  // grid (heads, query tiles, segments), the last query tile (most keys) first: CTAs are handed out
  // x-fastest, so the longest work starts first
  const int seg = blockIdx.z, h = blockIdx.x;
  const int q0 = seg_q_start[seg], qlen = seg_q_start[seg + 1] - q0;
  const int tile0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * 64;
  if (tile0 >= qlen) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tg = lane & 3;
  const int pos0 = seg_pos0[seg];
  const int kvh = h / (H / Hkv);
  const int* bt = block_table + (size_t)seg * max_blocks;
  const int rows_here = qlen - tile0 < 64 ? qlen - tile0 : 64;
  const int k_last = pos0 + tile0 + rows_here - 1;                 // last key any row of the tile sees
  int k_first = 0;
  if (window > 0) { const int f = pos0 + tile0 - window + 1; k_first = f > 0 ? f : 0; }
  const int tile_begin = k_first >> 6, tile_end = k_last >> 6;     // inclusive range of 64-key tiles
  const size_t page_elems = (size_t)2 * Hkv * page * HD;
  const size_t v_off = (size_t)Hkv * page * HD;

  // Q tile (rows beyond the segment are zero)
  for (int c = tid; c < 64 * CH; c += 128) {
    const int r = c / CH, ch = c - r * CH;
    bf16* dst = sQ + r * HD + ((ch ^ (r & 7)) << 3);
    if (r < rows_here) cp_async16(dst, q + (size_t)(q0 + tile0 + r) * ld_q + (size_t)h * HD + ch * 8);
    else *(uint4*)dst = make_uint4(0, 0, 0, 0);
  }
  auto load_kv = [&](int tile, int stage) {
    bf16* dk = sK + stage * 64 * HD;
    bf16* dv = sV + stage * 64 * HD;
    for (int c = tid; c < 64 * CH; c += 128) {
      const int r = c / CH, ch = c - r * CH;
      const int key = tile * 64 + r;
      const int off = r * HD + ((ch ^ (r & 7)) << 3);
      if (key <= k_last) {
        const bf16* src = cache + (size_t)bt[key / page] * page_elems + ((size_t)kvh * page + (key % page)) * HD + ch * 8;
        cp_async16(dk + off, src);
        cp_async16(dv + off, src + v_off);
      } else {                                       // keys nobody sees: zeros, so that 0 * x stays 0
        *(uint4*)(dk + off) = make_uint4(0, 0, 0, 0);
        *(uint4*)(dv + off) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  load_kv(tile_begin, 0);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  // Q fragments of this warp's 16 rows stay in registers
  uint32_t qa[KS][4];
  {
    const int r = warp * 16 + (lane & 15);
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int ch = ks * 2 + (lane >> 4);
      ldsm_x4(qa[ks], sQ + r * HD + ((ch ^ (r & 7)) << 3));
    }
  }
  const int row_lo = tile0 + warp * 16 + g, row_hi = row_lo + 8;
  int hi[2] = {row_lo < qlen ? pos0 + row_lo : -1, row_hi < qlen ? pos0 + row_hi : -1};
  int lo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) lo[r] = (window > 0 && hi[r] - window + 1 > 0) ? hi[r] - window + 1 : 0;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int warp_last = pos0 + tile0 + warp * 16 + 15;             // keys beyond this are masked for the whole warp

  for (int tile = tile_begin; tile <= tile_end; ++tile) {
    const int stage = (tile - tile_begin) & 1;
    if (tile + 1 <= tile_end) load_kv(tile + 1, stage ^ 1);        // the other stage was released by the barrier below
    cp_async_commit();
    const bf16* tK = sK + stage * 64 * HD;
    const bf16* tV = sV + stage * 64 * HD;
    const int base = tile * 64;
    if (base <= warp_last) {
      float s[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t kb[4];
          const int r = np * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int ch = ks * 2 + ((lane >> 3) & 1);
          ldsm_x4(kb, tK + r * HD + ((ch ^ (r & 7)) << 3));
          mma_bf16(s[2 * np], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[0], kb[1]);
          mma_bf16(s[2 * np + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[2], kb[3]);
        }
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const int key = base + 8 * j + 2 * tg + (e & 1);
          const float v = (key >= lo[r] && key <= hi[r]) ? s[j][e] * scale_log2 : -INFINITY;
          s[j][e] = v;
          mx[r] = fmaxf(mx[r], v);
        }
      float corr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m[r], mx[r]);
        corr[r] = (m_new == -INFINITY) ? 1.f : exp2f(m[r] - m_new);
        m[r] = m_new;
        l[r] *= corr[r];
      }
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0];
        o[i][2] *= corr[1]; o[i][3] *= corr[1];
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        uint32_t pa[4];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float e[4];
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const float sv = s[2 * kk + half][x];
            e[x] = (sv == -INFINITY) ? 0.f : exp2f(sv - m[x >> 1]);
            l[x >> 1] += e[x];
          }
          pa[2 * half] = pack_bf16(e[0], e[1]);
          pa[2 * half + 1] = pack_bf16(e[2], e[3]);
        }
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
          uint32_t vb[4];
          const int r = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int ch = dp * 2 + (lane >> 4);
          ldsm_x4_trans(vb, tV + r * HD + ((ch ^ (r & 7)) << 3));
          mma_bf16(o[2 * dp], pa[0], pa[1], pa[2], pa[3], vb[0], vb[1]);
          mma_bf16(o[2 * dp + 1], pa[0], pa[1], pa[2], pa[3], vb[2], vb[3]);
        }
      }
    }
    cp_async_wait<0>();
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r ? row_hi : row_lo;
    if (row >= qlen) continue;
    const float inv = 1.f / l[r];
    bf16* orow = out + (size_t)(q0 + row) * ld_out + (size_t)h * HD;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
      *(uint32_t*)(orow + i * 8 + 2 * tg) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
  }
}

template <int HD>
int launch_prefill_tile(bf16* out, int ld_out, const bf16* q, int ld_q, const bf16* cache, const int* seg_q_start, const int* seg_pos0,
                        const int* bt, int max_blocks, int S, int max_q_len, int H, int Hkv, int page, int window, float scale_log2,
                        cudaStream_t st) {
  constexpr int smem = (64 + 4 * 64) * HD * 2;
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tile_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(H, (max_q_len + 63) / 64, S);
  return qv_launch(attn_prefill_tile_kernel<HD>, grid, dim3(128), (size_t)smem, st, out, ld_out, q, ld_q, cache, seg_q_start, seg_pos0,
                   bt, max_blocks, H, Hkv, page, window, scale_log2);
}

// ---------------------------------------------------------------- decode
// partial results of a slice: [token][head][slice][HD + 2] floats (out unnormalised, then m, l)
template <int HD, int ROWS>
__global__ void __launch_bounds__(128) attn_decode_kernel(bf16* __restrict__ out, int ld_out, const bf16* __restrict__ q, int ld_q,
                                                          const bf16* __restrict__ cache, const int* __restrict__ tok_pos,
                                                          const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                                                          int max_blocks, int H, int Hkv, int page, int window, float scale_log2,
                                                          int splits, float* __restrict__ partial) {
  extern __shared__ float sm[];                 // [4 warps][16 rows][HD + 2]
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.z, kvh = blockIdx.y, split = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const int G = H / Hkv;
  const int pos = tok_pos[t];
  const int* bt = block_table + (size_t)tok_seg[t] * max_blocks;
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int start = first & ~15;
  const int total = pos + 1 - start;
  int chunk = (total + splits - 1) / splits;
  chunk = (chunk + 63) & ~63;
  const int k_begin = start + split * chunk;
  int k_stop = k_begin + chunk;                  // exclusive
  if (k_stop > pos + 1) k_stop = pos + 1;
  const bf16* qtok = q + (size_t)t * ld_q + (size_t)kvh * G * HD;
  QFrag<HD, ROWS> qf;
  load_q<HD, ROWS>(qf, g < G ? qtok + (size_t)g * HD : nullptr, g + 8 < G ? qtok + (size_t)(g + 8) * HD : nullptr, tg);
  const int lo[2] = {first, first};
  const int hi[2] = {g < G ? pos : -1, g + 8 < G ? pos : -1};
  RowState<HD, ROWS> st;
  st.init();
  const size_t page_elems = (size_t)2 * Hkv * page * HD;
  const size_t v_off = (size_t)Hkv * page * HD;
  for (int base = k_begin + 16 * warp; base < k_stop; base += 64) {
    const bf16* kblk = cache + (size_t)bt[base / page] * page_elems + ((size_t)kvh * page + (base % page)) * HD;
    block16<HD, true, ROWS>(st, qf, kblk, kblk + v_off, base, lo, hi, scale_log2, g, tg);
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
    st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
  }
  // each warp leaves its rows in shared memory
  constexpr int ROW = HD + 2;
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int row = g + 8 * r;
    if (row >= G) continue;
    float* dst = sm + ((size_t)warp * 16 + row) * ROW;
#pragma unroll
    for (int i = 0; i < Shape<HD>::NT; ++i) {
      dst[out_dim<HD>(i, 2 * tg)] = st.o[i][2 * r];
      dst[out_dim<HD>(i, 2 * tg + 1)] = st.o[i][2 * r + 1];
    }
    if (tg == 0) { dst[HD] = st.m[r]; dst[HD + 1] = st.l[r]; }
  }
  __syncthreads();
  // merge the 4 warps in a fixed order (warp 0, 1, 2, 3)
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int row = idx / HD, d = idx - row * HD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, sm[((size_t)w * 16 + row) * ROW + HD]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* src = sm + ((size_t)w * 16 + row) * ROW;
      const float f = (src[HD] == -INFINITY) ? 0.f : exp2f(src[HD] - m);
      acc += src[d] * f;
      l += src[HD + 1] * f;
    }
    const int h = kvh * G + row;
    if (splits == 1) {
      out[(size_t)t * ld_out + (size_t)h * HD + d] = __float2bfloat16_rn(acc / l);
    } else {
      float* dst = partial + (((size_t)t * H + h) * splits + split) * ROW;
      dst[d] = acc;
      if (d == 0) { dst[HD] = m; dst[HD + 1] = l; }
    }
  }
}

// The same slice of work with the keys and values brought into shared memory by the copy engine:
// one thread requests, for every block of 16 keys, the kv head's 16 key rows and 16 value rows of
// the page (two contiguous copies of 16 * HD * 2 bytes) into a ring of stages; the four consumer
// warps take alternate blocks from the ring.  Per-thread loads keep too few bytes in flight to
// pull the cache at HBM speed (a 16-key block cost a warp ~3 us); bulk copies do not go through
// the load/store unit's miss queue.  Waits are bounded; a wait that gives up records a code in *err.
// ROWS = 1 when at most 8 query heads share a kv head (the lower half of the MMA tile); NW consumer warps.
#define DEC_STAGES 8
template <int HD, int ROWS, int NW>
__global__ void __launch_bounds__(32 * (NW + 1)) attn_decode_bulk_kernel(bf16* __restrict__ out, int ld_out, const bf16* __restrict__ q, int ld_q,
                                                               const bf16* __restrict__ cache, const int* __restrict__ tok_pos,
                                                               const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                                                               int max_blocks, int H, int Hkv, int page, int window, float scale_log2,
                                                               int splits, float* __restrict__ partial, int* err) {
  extern __shared__ uint8_t dec_smem[];
  constexpr int KB = 16 * HD * 2;                       // bytes of 16 key rows (and of 16 value rows)
  constexpr int STAGE = 2 * KB;
  constexpr int ROW = HD + 2;
  constexpr int RING = DEC_STAGES * STAGE, SCRATCH = NW * 8 * ROWS * ROW * 4;
  uint8_t* ring = (uint8_t*)(((uintptr_t)dec_smem + 127) & ~(uintptr_t)127);
  float* sm = (float*)ring;                             // the merge reuses the ring once it is drained
  uint64_t* full = (uint64_t*)(ring + (RING > SCRATCH ? RING : SCRATCH));
  uint64_t* empty = full + DEC_STAGES;
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.z, kvh = blockIdx.y, split = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  if (threadIdx.x == 0) {
    for (int s = 0; s < DEC_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  const int G = H / Hkv;
  const int pos = tok_pos[t];
  const int* bt = block_table + (size_t)tok_seg[t] * max_blocks;
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int start = first & ~15;
  const int total = pos + 1 - start;
  int chunk = (total + splits - 1) / splits;
  chunk = (chunk + 63) & ~63;
  const int k_begin = start + split * chunk;
  int k_stop = k_begin + chunk;                  // exclusive
  if (k_stop > pos + 1) k_stop = pos + 1;
  const int nblk = k_stop > k_begin ? (k_stop - k_begin + 15) >> 4 : 0;
  RowState<HD, ROWS> st;
  st.init();
  if (warp == NW) {
    if (lane == 0) {
      const size_t page_elems = (size_t)2 * Hkv * page * HD;
      const size_t v_off = (size_t)Hkv * page * HD;
      int pg = k_begin / page, in_pg = k_begin - pg * page;
      for (int i = 0; i < nblk; ++i) {
        const int s = i % DEC_STAGES;
        if (!mbar_wait(&empty[s], ((i / DEC_STAGES) & 1) ^ 1, err, 31)) break;
        const bf16* kblk = cache + (size_t)bt[pg] * page_elems + ((size_t)kvh * page + in_pg) * HD;
        mbar_expect_tx(&full[s], STAGE);
        bulk_load_1d(ring + (size_t)s * STAGE, kblk, &full[s], KB);
        bulk_load_1d(ring + (size_t)s * STAGE + KB, kblk + v_off, &full[s], KB);
        in_pg += 16;
        if (in_pg == page) { in_pg = 0; ++pg; }
      }
    }
  } else {
    const bf16* qtok = q + (size_t)t * ld_q + (size_t)kvh * G * HD;
    QFrag<HD, ROWS> qf;
    load_q<HD, ROWS>(qf, g < G ? qtok + (size_t)g * HD : nullptr, g + 8 < G ? qtok + (size_t)(g + 8) * HD : nullptr, tg);
    const int lo[2] = {first, first};
    const int hi[2] = {g < G ? pos : -1, g + 8 < G ? pos : -1};
    for (int i = warp; i < nblk; i += NW) {
      const int s = i % DEC_STAGES;
      int ok = 1;
      if (lane == 0) ok = mbar_wait(&full[s], (i / DEC_STAGES) & 1, err, 32) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      const bf16* kblk = (const bf16*)(ring + (size_t)s * STAGE);
      block16<HD, true, ROWS>(st, qf, kblk, kblk + 16 * HD, k_begin + 16 * i, lo, hi, scale_log2, g, tg);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
      st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
    }
  }
  __syncthreads();                              // every block is consumed: the ring is free for the merge
  if (warp < NW) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int row = g + 8 * r;
      if (row >= G) continue;
      float* dst = sm + ((size_t)warp * 8 * ROWS + row) * ROW;
#pragma unroll
      for (int i = 0; i < Shape<HD>::NT; ++i) {
        dst[out_dim<HD>(i, 2 * tg)] = st.o[i][2 * r];
        dst[out_dim<HD>(i, 2 * tg + 1)] = st.o[i][2 * r + 1];
      }
      if (tg == 0) { dst[HD] = st.m[r]; dst[HD + 1] = st.l[r]; }
    }
  }
  __syncthreads();
  // merge the warps in a fixed order (warp 0, 1, 2, ...)
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int row = idx / HD, d = idx - row * HD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) m = fmaxf(m, sm[((size_t)w * 8 * ROWS + row) * ROW + HD]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float* src = sm + ((size_t)w * 8 * ROWS + row) * ROW;
      const float f = (src[HD] == -INFINITY) ? 0.f : exp2f(src[HD] - m);
      acc += src[d] * f;
      l += src[HD + 1] * f;
    }
    const int h = kvh * G + row;
    if (splits == 1) {
      out[(size_t)t * ld_out + (size_t)h * HD + d] = __float2bfloat16_rn(acc / l);
    } else {
      float* dst = partial + (((size_t)t * H + h) * splits + split) * ROW;
      dst[d] = acc;
      if (d == 0) { dst[HD] = m; dst[HD + 1] = l; }
    }
  }
}

// merges the slices of one (token, head) in slice order
__global__ void attn_combine_kernel(bf16* __restrict__ out, int ld_out, const float* __restrict__ partial, int H, int hd, int splits) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.y, h = blockIdx.x;
  const int row = hd + 2;
  const float* src = partial + ((size_t)t * H + h) * splits * row;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, src[(size_t)s * row + hd]);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f, l = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = src[(size_t)s * row + hd];
      const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
      acc += src[(size_t)s * row + d] * f;
      l += src[(size_t)s * row + hd + 1] * f;
    }
    out[(size_t)t * ld_out + (size_t)h * hd + d] = __float2bfloat16_rn(acc / l);
  }
}

template <int HD>
int launch_prefill(bf16* out, int ld_out, const bf16* q, int ld_q, const bf16* cache, const int* seg_q_start, const int* seg_pos0,
                   const int* bt, int max_blocks, int S, int max_q_len, int H, int Hkv, int page, int window, float scale_log2,
                   cudaStream_t st) {
  dim3 grid(H, (max_q_len + 63) / 64, S);
  return qv_launch(attn_prefill_kernel<HD>, grid, dim3(128), 0, st, out, ld_out, q, ld_q, cache, seg_q_start, seg_pos0, bt,
                   max_blocks, H, Hkv, page, window, scale_log2);
}

// 0: keys and values through the copy engine into shared memory (needs the error word); 1: per-thread loads
int g_decode_variant = 0;
int* g_decode_err = nullptr;

template <int HD>
int launch_decode(bf16* out, int ld_out, const bf16* q, int ld_q, const bf16* cache, const int* tok_pos, const int* tok_seg,
                  const int* bt, int max_blocks, int T, int H, int Hkv, int page, int window, float scale_log2, int splits,
                  float* partial, cudaStream_t st) {
  dim3 grid(splits, Hkv, T);
  int rc;
  if (g_decode_variant == 0 && g_decode_err != nullptr) {
    // at most 8 query heads per kv head: half-tile state (fewer registers, fewer instructions)
    const int G = H / Hkv;
#define BULK_LAUNCH(ROWS_, NW_)                                                                                          \
  do {                                                                                                                   \
    constexpr int ring = DEC_STAGES * 2 * 16 * HD * 2, scratch = NW_ * 8 * ROWS_ * (HD + 2) * 4;                         \
    const size_t smem = (size_t)(ring > scratch ? ring : scratch) + 2 * DEC_STAGES * 8 + 128;                            \
    static bool configured = false;                                                                                      \
    if (!configured && smem > 48 * 1024) {                                                                               \
      cudaError_t e = cudaFuncSetAttribute(attn_decode_bulk_kernel<HD, ROWS_, NW_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                                               \
      configured = true;                                                                                                 \
    }                                                                                                                    \
    rc = qv_launch(attn_decode_bulk_kernel<HD, ROWS_, NW_>, grid, dim3(32 * (NW_ + 1)), smem, st, out, ld_out, q, ld_q, cache, tok_pos, \
                   tok_seg, bt, max_blocks, H, Hkv, page, window, scale_log2, splits, partial, g_decode_err);           \
  } while (0)
    if (G > 8) BULK_LAUNCH(2, 4);
    else BULK_LAUNCH(1, 4);
#undef BULK_LAUNCH
  } else {
    const size_t smem = (size_t)4 * 16 * (HD + 2) * sizeof(float);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    // (the half-tile state that helps the bulk kernel measured slower here: 14.8 against 13.6 us)
    rc = qv_launch(attn_decode_kernel<HD, 2>, grid, dim3(128), smem, st, out, ld_out, q, ld_q, cache, tok_pos, tok_seg, bt,
                   max_blocks, H, Hkv, page, window, scale_log2, splits, partial);
  }
  if (rc || splits == 1) return rc;
  return qv_launch(attn_combine_kernel, dim3(H, T), dim3(HD < 128 ? 64 : 128), 0, st, out, ld_out, (const float*)partial, H,
                   (int)HD, splits);
}

}  // namespace

#define FOR_HEAD_DIMS(X) X(16) X(32) X(48) X(64) X(80) X(96) X(112) X(128)

// Which decode kernel runs (0: shared-memory ring filled by bulk copies, the default once the error
// word is set; 1: per-thread loads), and the device word that bounded waits report into.
extern "C" void qv_attn_set_decode_variant(int v) { g_decode_variant = v; }
extern "C" void qv_attn_set_error_word(int* err) { g_decode_err = err; }

// Floats of workspace that qv_attn_decode_bf16 needs for `splits` > 1.
extern "C" long long qv_attn_decode_workspace_floats(int T, int H, int hd, int splits) {
  return splits > 1 ? (long long)T * H * splits * (hd + 2) : 0;
}

// Prompt portions (any mix of segments).  Refuses head sizes other than 16..128 in steps of 16,
// pages that are no multiple of 16, and operands that are not 16-byte aligned row by row.
extern "C" int qv_attn_prefill_bf16(void* out, int ld_out, const void* q, int ld_q, const void* cache, const int* seg_q_start,
                                    const int* seg_pos0, const int* block_table, int max_blocks, int S, int max_q_len, int H,
                                    int Hkv, int hd, int page, int window, float scale, int variant, void* stream) {
  // variant 0: the shared-memory kernel where it exists (head sizes 64 and 128), else the
  // register-direct one; variant 1: always the register-direct kernel.
  if (S <= 0 || max_q_len <= 0) return 0;
  if (Hkv <= 0 || H % Hkv || page % 16 || (ld_q & 7) || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15)) return QV_ERR_UNSUPPORTED;
  if (S > 65535 || (max_q_len + 63) / 64 > 65535) return QV_ERR_TOO_LARGE;
  const float sl2 = scale * 1.4426950408889634f;
  if ((hd == 64 || hd == 128) && (ld_out & 1) == 0 && variant == 0) {
    if (hd == 64)
      return launch_prefill_tile<64>((bf16*)out, ld_out, (const bf16*)q, ld_q, (const bf16*)cache, seg_q_start, seg_pos0,
                                     block_table, max_blocks, S, max_q_len, H, Hkv, page, window, sl2, (cudaStream_t)stream);
    return launch_prefill_tile<128>((bf16*)out, ld_out, (const bf16*)q, ld_q, (const bf16*)cache, seg_q_start, seg_pos0,
                                    block_table, max_blocks, S, max_q_len, H, Hkv, page, window, sl2, (cudaStream_t)stream);
  }
#define CASE(D)                                                                                                          \
  if (hd == D)                                                                                                           \
    return launch_prefill<D>((bf16*)out, ld_out, (const bf16*)q, ld_q, (const bf16*)cache, seg_q_start, seg_pos0, block_table, \
                             max_blocks, S, max_q_len, H, Hkv, page, window, sl2, (cudaStream_t)stream);
  FOR_HEAD_DIMS(CASE)
#undef CASE
  return QV_ERR_UNSUPPORTED;
}

// One query row per token (decoded tokens; also right, if slow, for any token of a portion).
// The query heads of one kv head form the MMA tile, so H / Hkv must not exceed 16.
extern "C" int qv_attn_decode_bf16(void* out, int ld_out, const void* q, int ld_q, const void* cache, const int* tok_pos,
                                   const int* tok_seg, const int* block_table, int max_blocks, int T, int H, int Hkv, int hd,
                                   int page, int window, float scale, int splits, float* partial, void* stream) {
  if (T <= 0) return 0;
  if (Hkv <= 0 || H % Hkv || H / Hkv > 16 || page % 16 || (ld_q & 7) || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15))
    return QV_ERR_UNSUPPORTED;
  if (splits < 1 || (splits > 1 && !partial) || T > 65535 || Hkv > 65535) return QV_ERR_UNSUPPORTED;
  const float sl2 = scale * 1.4426950408889634f;
#define CASE(D)                                                                                                         \
  if (hd == D)                                                                                                          \
    return launch_decode<D>((bf16*)out, ld_out, (const bf16*)q, ld_q, (const bf16*)cache, tok_pos, tok_seg, block_table, \
                            max_blocks, T, H, Hkv, page, window, sl2, splits, partial, (cudaStream_t)stream);
  FOR_HEAD_DIMS(CASE)
#undef CASE
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- decode without allocation
// See attention_noalloc.h.  The workspace of the key slices is this array; host code may not
// use its name as a pointer (on the host the name stands for a shadow object, not for device
// memory), so the device address is looked up once per device and handed to the kernel.
#include "attention_noalloc.h"

static __device__ __align__(256) float g_decode_scratch[QV_ATTN_STATIC_SCRATCH_FLOATS];

#define QV_MAX_DEVICES 64
static float* g_decode_scratch_addr[QV_MAX_DEVICES];     // per device, filled on that device's first call

extern "C" int qv_attn_decode_bf16_static(void* out, int ld_out, const void* q, int ld_q, const void* cache, const int* tok_pos,
                                          const int* tok_seg, const int* block_table, int max_blocks, int T, int H, int Hkv,
                                          int hd, int page, int window, float scale, int splits, void* stream) {
  if (T <= 0) return 0;
  if (splits < 1) return QV_ERR_UNSUPPORTED;
  if (splits > 1 && (long long)T * H * splits * (hd + 2) > (long long)QV_ATTN_STATIC_SCRATCH_FLOATS)
    return QV_ERR_STATIC_SCRATCH_TOO_SMALL;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= QV_MAX_DEVICES) return QV_ERR_UNSUPPORTED;
  if (g_decode_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_decode_scratch);    // the address on the current device
    if (e != cudaSuccess) return (int)e;
    g_decode_scratch_addr[dev] = p;
  }
  return qv_attn_decode_bf16(out, ld_out, q, ld_q, cache, tok_pos, tok_seg, block_table, max_blocks, T, H, Hkv, hd, page,
                             window, scale, splits, g_decode_scratch_addr[dev], stream);
}

extern "C" const char* qv_attn_decode_static_strerror(int code) {
  if (code == 0) return "ok";
  if (code == QV_ERR_STATIC_SCRATCH_TOO_SMALL)
    return "T * H * splits * (head_dim + 2) exceeds the library's built-in workspace (QV_ATTN_STATIC_SCRATCH_FLOATS); "
           "use fewer slices or tokens per call, or qv_attn_decode_bf16 with a workspace of your own";
  if (code == QV_ERR_UNSUPPORTED) return "sizes or alignment this kernel does not take";
  if (code == QV_ERR_TOO_LARGE) return "too many tokens or heads for one launch";
  return cudaGetErrorString((cudaError_t)code);
}
