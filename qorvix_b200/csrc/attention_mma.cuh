// Blocks of 16 keys on mma.sync m16n8k16 with an online softmax in float32, operands loaded
// from global memory straight into MMA fragments; shared by the attention kernels.
#pragma once
#include "common.cuh"

namespace {

__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&h;
}

template <int N> struct Words { uint32_t w[N]; };
template <int N> __device__ __forceinline__ Words<N> load_words(const bf16* p);
template <> __device__ __forceinline__ Words<4> load_words<4>(const bf16* p) {
  const uint4 v = *(const uint4*)p; Words<4> r; r.w[0] = v.x; r.w[1] = v.y; r.w[2] = v.z; r.w[3] = v.w; return r;
}
template <> __device__ __forceinline__ Words<2> load_words<2>(const bf16* p) {
  const uint2 v = *(const uint2*)p; Words<2> r; r.w[0] = v.x; r.w[1] = v.y; return r;
}
template <> __device__ __forceinline__ Words<1> load_words<1>(const bf16* p) {
  Words<1> r; r.w[0] = *(const uint32_t*)p; return r;
}

// Sizes that follow from the head size.
template <int HD> struct Shape {
  static constexpr int KW = (HD % 32 == 0) ? 4 : 2;       // 32-bit words per thread per K/Q load
  static constexpr int KCH = HD / (KW * 8);               // chunks of KW*8 dims along the dot product
  static constexpr int VW = (HD % 64 == 0) ? 4 : ((HD % 32 == 0) ? 2 : 1);   // words per thread per V load
  static constexpr int VCH = HD / (VW * 16);              // chunks of VW*16 output dims
  static constexpr int NT = HD / 8;                       // output n-tiles
};

// Q rows g and g+8 of a 16-row tile as A fragments, in the k order of the K loads.
// ROWS = 1: only rows 0..7 of the tile are real (at most 8 query rows); the fragments, the running
// state and the outputs of rows 8..15 are then not kept at all, which frees ~48 registers.
template <int HD, int ROWS = 2> struct QFrag { uint32_t w[Shape<HD>::KCH][ROWS][Shape<HD>::KW]; };

template <int HD, int ROWS = 2>
__device__ __forceinline__ void load_q(QFrag<HD, ROWS>& q, const bf16* row_lo, const bf16* row_hi, int tg) {
  constexpr int KW = Shape<HD>::KW;
#pragma unroll
  for (int c = 0; c < Shape<HD>::KCH; ++c) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const bf16* p = r ? row_hi : row_lo;
      if (p) {
        Words<KW> v = load_words<KW>(p + c * KW * 8 + tg * KW * 2);
#pragma unroll
        for (int i = 0; i < KW; ++i) q.w[c][r][i] = v.w[i];
      } else {
#pragma unroll
        for (int i = 0; i < KW; ++i) q.w[c][r][i] = 0u;
      }
    }
  }
}

// Running softmax state of rows g and g+8 and their output fragments.
template <int HD, int ROWS = 2> struct RowState {
  float m[ROWS], l[ROWS];
  float o[Shape<HD>::NT][2 * ROWS];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) { m[r] = -INFINITY; l[r] = 0.f; }
#pragma unroll
    for (int i = 0; i < Shape<HD>::NT; ++i)
#pragma unroll
      for (int e = 0; e < 2 * ROWS; ++e) o[i][e] = 0.f;
  }
};

// One block of 16 keys starting at absolute key index `base` (a multiple of 16).
// kpage / vpage: this kv head's K and V rows of the page that holds the block, at the block's
// first key.  Row r in {0,1} (tile rows g, g+8) sees keys in [lo[r], hi[r]] (inclusive).
// EARLY_V: the V rows are requested together with the K rows, before the scores are formed,
// so that both round trips to memory overlap (decode, where latency is what costs).
template <int HD, bool EARLY_V, int ROWS = 2>
__device__ __forceinline__ void block16(RowState<HD, ROWS>& st, const QFrag<HD, ROWS>& q, const bf16* __restrict__ kblk,
                                        const bf16* __restrict__ vblk, int base, const int* lo, const int* hi,
                                        float scale_log2, int g, int tg) {
  constexpr int KW = Shape<HD>::KW, KCH = Shape<HD>::KCH, VW = Shape<HD>::VW, VCH = Shape<HD>::VCH;
  float s[2][4];
  Words<KW> kw[2][KCH];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const bf16* krow = kblk + (size_t)(8 * j + g) * HD + tg * KW * 2;
#pragma unroll
    for (int c = 0; c < KCH; ++c) kw[j][c] = load_words<KW>(krow + c * KW * 8);
  }
  const bf16* v0 = vblk + (size_t)(2 * tg) * HD + g * VW * 2;
  Words<VW> vw[VCH][4];
  if (EARLY_V) {
#pragma unroll
    for (int c = 0; c < VCH; ++c) {
      vw[c][0] = load_words<VW>(v0 + c * VW * 16);
      vw[c][1] = load_words<VW>(v0 + HD + c * VW * 16);
      vw[c][2] = load_words<VW>(v0 + 8 * HD + c * VW * 16);
      vw[c][3] = load_words<VW>(v0 + 9 * HD + c * VW * 16);
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int c = 0; c < KCH; ++c) {
#pragma unroll
      for (int step = 0; step < KW / 2; ++step) {
        // with ROWS == 1 rows 8..15 of the tile are zero: their fragments are the constant 0
        const uint32_t a1 = ROWS == 2 ? q.w[c][ROWS - 1][2 * step] : 0u, a3 = ROWS == 2 ? q.w[c][ROWS - 1][2 * step + 1] : 0u;
        mma_bf16(s[j], q.w[c][0][2 * step], a1, q.w[c][0][2 * step + 1], a3, kw[j][c].w[2 * step], kw[j][c].w[2 * step + 1]);
      }
    }
  }
  // mask, running maximum
  float mx[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) mx[r] = -INFINITY;
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int e = 0; e < 2 * ROWS; ++e) {
      const int r = e >> 1;
      const int key = base + 8 * j + 2 * tg + (e & 1);
      const float v = (key >= lo[r] && key <= hi[r]) ? s[j][e] * scale_log2 : -INFINITY;
      s[j][e] = v;
      mx[r] = fmaxf(mx[r], v);
    }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
  }
  float corr[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const float m_new = fmaxf(st.m[r], mx[r]);
    // a row with no visible key so far keeps m = -inf; exp2(-inf - (-inf)) must not be formed
    corr[r] = (m_new == -INFINITY) ? 1.f : exp2f(st.m[r] - m_new);
    st.m[r] = m_new;
    st.l[r] *= corr[r];
  }
  uint32_t p[4];     // A fragment of P: a0 (row g, keys 2tg..), a1 (row g+8), a2 (row g, keys 8+2tg..), a3
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    float e[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int x = 0; x < 2 * ROWS; ++x) {
      const int r = x >> 1;
      e[x] = (s[j][x] == -INFINITY) ? 0.f : exp2f(s[j][x] - st.m[r]);
      st.l[r] += e[x];
    }
    p[2 * j] = pack_bf16(e[0], e[1]);
    p[2 * j + 1] = ROWS == 2 ? pack_bf16(e[2], e[3]) : 0u;
  }
#pragma unroll
  for (int i = 0; i < Shape<HD>::NT; ++i) {
#pragma unroll
    for (int e = 0; e < 2 * ROWS; ++e) st.o[i][e] *= corr[e >> 1];
  }
  // P.V: this thread supplies keys 2tg, 2tg+1, 8+2tg, 9+2tg for output column n = g of each n-tile;
  // n-tile e of chunk c is head dim c*VW*16 + g*VW*2 + e.
#pragma unroll
  for (int c = 0; c < VCH; ++c) {
    if (!EARLY_V) {
      vw[c][0] = load_words<VW>(v0 + c * VW * 16);
      vw[c][1] = load_words<VW>(v0 + HD + c * VW * 16);
      vw[c][2] = load_words<VW>(v0 + 8 * HD + c * VW * 16);
      vw[c][3] = load_words<VW>(v0 + 9 * HD + c * VW * 16);
    }
#pragma unroll
    for (int e = 0; e < VW * 2; ++e) {
      const int w = e >> 1;
      const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
      const uint32_t b0 = __byte_perm(vw[c][0].w[w], vw[c][1].w[w], sel);
      const uint32_t b1 = __byte_perm(vw[c][2].w[w], vw[c][3].w[w], sel);
      if (ROWS == 2) {
        mma_bf16(st.o[c * VW * 2 + e], p[0], p[1], p[2], p[3], b0, b1);
      } else {
        // rows 8..15 are not kept: their accumulators go in as zero and come out unused
        float d[4] = {st.o[c * VW * 2 + e][0], st.o[c * VW * 2 + e][1], 0.f, 0.f};
        mma_bf16(d, p[0], 0u, p[2], 0u, b0, b1);
        st.o[c * VW * 2 + e][0] = d[0];
        st.o[c * VW * 2 + e][1] = d[1];
      }
    }
  }
}

// Output fragment (n-tile index i = c*VW*2 + e, column n) -> head dim.
template <int HD> __device__ __forceinline__ int out_dim(int i, int n) {
  constexpr int VW = Shape<HD>::VW;
  const int c = i / (VW * 2), e = i - c * VW * 2;
  return c * VW * 16 + n * VW * 2 + e;
}

}  // namespace
