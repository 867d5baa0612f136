// All layers of a decode step (a few tokens, one per request) as ONE persistent kernel.
//
// A decode step is bound by reading the weights once from HBM.  Run as one kernel per
// operation (the reference's forward is ~10 launches per layer, cuda/src/cuda_backend.cu:1380-1440),
// every product pays a ramp-up and a tail in which HBM idles: the next kernel cannot request its
// weights before the one ahead has given up its shared memory.  Here one CTA per SM stays
// resident for the whole step and keeps a ring of weight tiles (TMA, 128-byte swizzle) full
// across operation boundaries: while the CTAs meet at a grid barrier, or work through the
// attention of a layer, the weight stream of the next product is already in flight.
//
//   warp 0      requests weight tiles, running ahead through all products of all layers
//   warp 1      issues tcgen05.mma (128 weight rows x BN tokens x 64 k per stage), accumulators
//               double-buffered in tensor memory
//   warps 4-11  workers: during a product four of them drain accumulators and four copy the
//               activation tiles into the stages; between products all run the element-wise
//               steps (residual add + RMS norm, rotary + cache write, attention over the pages,
//               merge of the key slices, SiLU gate) spread over all CTAs
//
// Every product is cut into (row tile, k block) units that are dealt out evenly and contiguously
// to the CTAs (so a CTA may own a part of a tile's reduction).  Each part leaves its partial sums
// in a float32 workspace; whoever consumes the product adds the parts of a tile in part order, so
// the result does not depend on timing.  Steps are separated by a grid barrier (one atomic
// counter, bounded spin).  Data produced inside the kernel is read past L1 (ld.global.cg / TMA).
//
// Every wait is bounded.  A wait that gives up records a code in *err, raises the CTA's abort
// flag, and from then on every role skips its work but keeps taking the CTA's barriers, so the
// kernel winds down (tensor memory freed, outstanding copies awaited) instead of hanging.
#include "tc_common.cuh"
#include "attention_mma.cuh"

#define FUSED_THREADS 384
#define FUSED_WORKERS 256            // warps 4..11
#define FUSED_MAX_STAGES 16
#define X_LOADER_WARPS 4             // worker warps 4..7 bring in the activation tiles
#define W_TILE_BYTES (BM * BK * 2)
#define GRID_SPIN_LIMIT (1u << 22)
#define FUSED_MAX_TILES 4096         // row tiles of a layer's four products together

struct FusedHostLayer {        // what the caller gives for one layer: 8-byte fields only
  const void* w[4];
  long long n[4];
  long long k[4];
  const float* norm1;
  const float* norm2;
  void* cache;
  const int* block_table;
  const void* rope;            // float32 [rope_rows][rot/2][2], or null
  double eps1, eps2, scale;
  long long window, rot, rope_rows, interleaved;
};

struct FusedHostArgs {         // 8-byte fields only
  const void* layers;          // device array of FusedLayer
  const float* final_norm;
  float* resid;
  void* x_norm; void* q_buf; void* attn_out; void* act;
  float* ws[4];
  float* attn_partial;
  float* ssq;
  const int* tok_pos; const int* tok_seg;
  unsigned* barrier; int* err;
  long long num_layers, M, BN, d, H, Hkv, hd, f, page, max_blocks, splits;
  double final_eps;
};

namespace {

struct alignas(64) FusedLayer {
  CUtensorMap w[4];          // qkv, o, gate/up (rows interleaved by 16), down: box 128 rows x 64 k
  int n[4];                  // rows of each matrix
  int k[4];                  // reduction length of each
  int max_parts[4];          // most CTAs that share one row tile of each product
  const float* norm1;        // weight of the norm before the mixer
  const float* norm2;        // ... before the feed-forward
  bf16* cache;               // this layer's pages [pages + 1, 2, Hkv, page, hd]
  const int* block_table;    // [rows, max_blocks] of the layer's cache group
  const float2* rope;        // [rope_rows][rot/2] (cos, sin); null: no rotation
  float eps1, eps2;
  float scale_log2;          // attention scale * log2(e)
  int window;
  int rot, rope_rows;
  int interleaved;           // gate/up rows interleaved by 16 (else: gate rows, then up rows)
};

struct FusedParams {
  const FusedLayer* layers;
  const float* final_norm;
  float* resid;                  // [M, d] residual stream, in and out
  bf16* x_norm;                  // [BN, d]   normalised input of the next product; on return: after the final norm
  bf16* q_buf;                   // [M, H*hd] rotated queries
  bf16* attn_out;                // [BN, H*hd]
  bf16* act;                     // [BN, f]
  float* ws[4];                  // partial sums of each product: [tile][part][BN tokens][128 rows]
  float* attn_partial;           // [M][H][splits][hd + 2]
  float* ssq;                    // [M][ceil(d/128)] sums of squares of the residual, chunk by chunk
  const int* tok_pos;
  const int* tok_seg;
  unsigned* barrier;
  int* err;
  long long* trace;              // optional: [step][CTA] time at which the CTA left the step's barrier
  int num_layers, M, d, H, Hkv, hd, f, page, max_blocks, splits, stages;
  float final_eps;
};

// Units u in [0, U) dealt to G CTAs: CTA c owns [share_begin(c), share_begin(c + 1)).
struct Share { int q, rem; };
__host__ __device__ inline Share make_share(int U, int G) { Share s; s.q = U / G; s.rem = U % G; return s; }
__host__ __device__ inline int share_begin(int c, Share s) { return c * s.q + (c < s.rem ? c : s.rem); }
__host__ __device__ inline int share_owner(int u, Share s) {
  const int lim = s.rem * (s.q + 1);
  return u < lim ? u / (s.q + 1) : s.rem + (u - lim) / s.q;
}

struct Product {           // one weight matrix as the CTAs see it
  int tiles, kbs, U;
  Share sh;
  __device__ __forceinline__ void set(int n, int k, int G) {
    tiles = (n + BM - 1) / BM; kbs = (k + BK - 1) / BK; U = tiles * kbs; sh = make_share(U, G);
  }
  // CTAs first..last hold the parts of tile t, in part order
  __device__ __forceinline__ int first_cta(int t) const { return share_owner(t * kbs, sh); }
  __device__ __forceinline__ int last_cta(int t) const { return share_owner((t + 1) * kbs - 1, sh); }
};

__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void worker_bar() { asm volatile("bar.sync 1, %0;" ::"n"(FUSED_WORKERS) : "memory"); }


struct Ctl {                       // shared-memory control block
  uint64_t full[FUSED_MAX_STAGES];
  uint64_t empty[FUSED_MAX_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_slot;
  volatile int abort;
  int part_off[4];                 // where each product's tiles start in part_count
  uint8_t part_count[FUSED_MAX_TILES];   // parts of every row tile of the current layer's products
};

__device__ __forceinline__ bool aborted(Ctl* c) { return c->abort != 0; }
__device__ __forceinline__ void give_up(Ctl* c, int* err, int code) {
  atomicCAS(err, 0, code);
  c->abort = 1;
}
// Bounded wait that also ends when the CTA has given up elsewhere.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, Ctl* c, int* err, int code) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023) == 1023 && aborted(c)) return false;
  }
  give_up(c, err, code);
  return false;
}

// One thread per CTA: arrive, then wait until all CTAs have arrived `round` times.
__device__ __forceinline__ void grid_barrier(const FusedParams& p, Ctl* c, unsigned round) {
  if (aborted(c)) return;
  __threadfence();
  atomicAdd(p.barrier, 1u);
  const unsigned target = round * gridDim.x;
  for (uint32_t i = 0; i < GRID_SPIN_LIMIT; ++i) {
    if (ld_acquire(p.barrier) >= target) { __threadfence(); return; }
    if ((i & 255) == 255 && *(volatile int*)p.err != 0) { c->abort = 1; return; }
  }
  give_up(c, p.err, 20);
}


// The parts of one tile, as a consumer sees them: where the first part lies and how many there are.
struct Parts {
  const float* base;       // part 0 of the tile, token 0, row 0
  int count;
  size_t stride;           // floats between parts
};
// (the counts come from a table in shared memory, filled once per layer: finding them needs
// four integer divisions, too slow to repeat for every element)
__device__ __forceinline__ Parts parts_of(const float* ws, int mp, const Ctl* ctl, int gi, int t, int BN) {
  Parts q;
  q.count = ctl->part_count[ctl->part_off[gi] + t];
  q.stride = (size_t)BN * BM;
  q.base = ws + (size_t)t * mp * q.stride;
  return q;
}
// Sum over the parts, in part order, at (token, row .. row + 3).  The first eight loads are issued
// together (a tile rarely has more parts), so the sum costs one trip to L2, not one per part.
__device__ __forceinline__ float4 parts_sum4(const Parts& q, int tok, int r) {
  const float* src = q.base + (size_t)tok * BM + r;
  float4 v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = j < q.count ? __ldcg((const float4*)(src + j * q.stride)) : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 acc = v[0];
#pragma unroll
  for (int j = 1; j < 8; ++j) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
  for (int j = 8; j < q.count; ++j) {
    const float4 w = __ldcg((const float4*)(src + j * q.stride));
    acc.x += w.x; acc.y += w.y; acc.z += w.z; acc.w += w.w;
  }
  return acc;
}
__device__ __forceinline__ float parts_sum1(const Parts& q, int tok, int r) {
  const float* src = q.base + (size_t)tok * BM + r;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = j < q.count ? __ldcg(src + j * q.stride) : 0.f;
  float acc = v[0];
#pragma unroll
  for (int j = 1; j < 8; ++j) acc += v[j];
  for (int j = 8; j < q.count; ++j) acc += __ldcg(src + j * q.stride);
  return acc;
}

__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// 1/rms of a token's residual row from the per-chunk sums of squares the norm step left, summed
// in chunk order by the whole warp (every lane gets the result).
__device__ __forceinline__ float row_scale(const FusedParams& p, int tok, float eps, int lane) {
  const int chunks = (p.d + BM - 1) / BM;
  float s = 0.f;
  for (int c = lane; c < chunks; c += 32) s += __ldcg(p.ssq + (size_t)tok * chunks + c);
  s = warp_sum(s);
  return 1.0f / sqrtf(s / (float)p.d + eps);
}

// ------------------------------------------------------------------ worker steps
// The norm is split in two so that no step needs a whole row in one place.  This step: one warp =
// one (token, chunk of 128 features): residual += parts of the product before (if any);
// x_norm = residual * w WITHOUT the 1/rms factor; the chunk's sum of squares goes to ssq.  The
// product that reads x_norm is linear, so whoever consumes its parts multiplies by 1/rms of the
// token (row_scale).
template <int BN>
__device__ __forceinline__ void step_add_prenorm(const FusedParams& p, const Ctl* ctl, const float* ws, int mp, int gi, const float* w,
                                                 int gw, int GW, int lane) {
  const int chunks = (p.d + BM - 1) / BM;
  for (int item = gw; item < p.M * chunks; item += GW) {
    const int tok = item / chunks, c = item - tok * chunks;
    const int f = c * BM + 4 * lane;
    float ss = 0.f;
    if (f < p.d) {
      float* res = p.resid + (size_t)tok * p.d + f;
      float4 a = __ldcg((const float4*)res);
      if (ws) {
        const Parts q = parts_of(ws, mp, ctl, gi, c, BN);
        const float4 b = parts_sum4(q, tok, 4 * lane);
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        *(float4*)res = a;
      }
      ss = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
      const float4 wv = *(const float4*)(w + f);
      uint2 out;
      out.x = pack2_bf16(a.x * wv.x, a.y * wv.y);
      out.y = pack2_bf16(a.z * wv.z, a.w * wv.w);
      *(uint2*)(p.x_norm + (size_t)tok * p.d + f) = out;
    }
    ss = warp_sum(ss);
    if (lane == 0) p.ssq[(size_t)tok * chunks + c] = ss;
  }
}

// After the last layer the norm's output leaves the kernel, so it is formed in full:
// x_norm = residual * (1/rms) * w, from the residual and the sums of squares of the step before.
__device__ __forceinline__ void step_final_norm(const FusedParams& p, const float* w, float eps, int gw, int GW, int lane) {
  const int chunks = (p.d + BM - 1) / BM;
  for (int item = gw; item < p.M * chunks; item += GW) {
    const int tok = item / chunks, c = item - tok * chunks;
    const float scale = row_scale(p, tok, eps, lane);
    const int f = c * BM + 4 * lane;
    if (f < p.d) {
      const float4 a = __ldcg((const float4*)(p.resid + (size_t)tok * p.d + f));
      const float4 wv = *(const float4*)(w + f);
      uint2 out;
      out.x = pack2_bf16(a.x * scale * wv.x, a.y * scale * wv.y);
      out.y = pack2_bf16(a.z * scale * wv.z, a.w * scale * wv.w);
      *(uint2*)(p.x_norm + (size_t)tok * p.d + f) = out;
    }
  }
}

// q, k, v of every token from the parts of the qkv product (times the token's 1/rms); q and k
// rotated; k and v into the pages.  One warp = one (token, head slot).
template <int BN>
__device__ __forceinline__ void step_rope(const FusedParams& p, const Ctl* ctl, const FusedLayer& L, int gw, int GW, int lane) {
  const int slots = p.H + 2 * p.Hkv, hd = p.hd, half = L.rot >> 1;
  const float* ws = p.ws[0];
  const int mp = L.max_parts[0];
  for (int item = gw; item < p.M * slots; item += GW) {
    const int tok = item / slots, slot = item - tok * slots;
    const int pos = p.tok_pos[tok];
    const float scale = row_scale(p, tok, L.eps1, lane);
    const int f0 = slot * hd;
    bf16* dst;
    if (slot < p.H) {
      dst = p.q_buf + (size_t)tok * p.H * hd + f0;
    } else {
      const int pg = L.block_table[(size_t)p.tok_seg[tok] * p.max_blocks + pos / p.page];
      const size_t page_elems = (size_t)2 * p.Hkv * p.page * hd;
      const bool is_v = slot >= p.H + p.Hkv;
      const int kvh = slot - p.H - (is_v ? p.Hkv : 0);
      dst = L.cache + (size_t)pg * page_elems + (is_v ? (size_t)p.Hkv * p.page * hd : 0) + ((size_t)kvh * p.page + pos % p.page) * hd;
    }
    // a head's features lie in at most two tiles when hd <= 128; value(i) = feature f0 + i
    auto value = [&](int i) {
      const int f = f0 + i, t = f / BM;
      return parts_sum1(parts_of(ws, mp, ctl, 0, t, BN), tok, f - t * BM) * scale;
    };
    const bool rotate = slot < p.H + p.Hkv && L.rope != nullptr && half > 0;
    if (rotate) {
      const float2* cs = L.rope + (size_t)(pos < L.rope_rows ? pos : L.rope_rows - 1) * half;
      // half <= 64: at most two pairs per lane; all their loads are issued before any is used
      const int i0 = lane, i1 = lane + 32;
      const bool h0 = i0 < half, h1 = i1 < half;
      const float a0 = h0 ? value(i0) : 0.f, b0 = h0 ? value(i0 + half) : 0.f;
      const float a1 = h1 ? value(i1) : 0.f, b1 = h1 ? value(i1 + half) : 0.f;
      if (h0) {
        const float2 c = cs[i0];
        dst[i0] = __float2bfloat16_rn(a0 * c.x - b0 * c.y);
        dst[i0 + half] = __float2bfloat16_rn(a0 * c.y + b0 * c.x);
      }
      if (h1) {
        const float2 c = cs[i1];
        dst[i1] = __float2bfloat16_rn(a1 * c.x - b1 * c.y);
        dst[i1 + half] = __float2bfloat16_rn(a1 * c.y + b1 * c.x);
      }
      for (int i = L.rot + lane; i < hd; i += 32) dst[i] = __float2bfloat16_rn(value(i));
    } else {
      for (int i = lane; i < hd; i += 32) dst[i] = __float2bfloat16_rn(value(i));
    }
  }
}

template <int HD>
__device__ __forceinline__ void load_q_cg(QFrag<HD>& q, const bf16* row_lo, const bf16* row_hi, int tg) {
  constexpr int KW = Shape<HD>::KW;
#pragma unroll
  for (int c = 0; c < Shape<HD>::KCH; ++c) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const bf16* ptr = r ? row_hi : row_lo;
      if (ptr) {
        const bf16* src = ptr + c * KW * 8 + tg * KW * 2;
        if constexpr (KW == 4) {
          const uint4 v = __ldcg((const uint4*)src);
          q.w[c][r][0] = v.x; q.w[c][r][1] = v.y; q.w[c][r][2] = v.z; q.w[c][r][3] = v.w;
        } else {
          const uint2 v = __ldcg((const uint2*)src);
          q.w[c][r][0] = v.x; q.w[c][r][1] = v.y;
        }
      } else {
#pragma unroll
        for (int i = 0; i < KW; ++i) q.w[c][r][i] = 0u;
      }
    }
  }
}

// One warp = one (token, kv head, slice of the keys); its rows are the query heads of the kv head.
template <int HD>
__device__ __forceinline__ void step_attention(const FusedParams& p, const FusedLayer& L, int gw, int GW, int lane) {
  const int G = p.H / p.Hkv, splits = p.splits;
  const int g = lane >> 2, tg = lane & 3;
  constexpr int ROW = HD + 2;
  const size_t page_elems = (size_t)2 * p.Hkv * p.page * HD;
  const size_t v_off = (size_t)p.Hkv * p.page * HD;
  for (int item = gw; item < p.M * p.Hkv * splits; item += GW) {
    const int split = item % splits;
    const int rest = item / splits;
    const int kvh = rest % p.Hkv, t = rest / p.Hkv;
    const int pos = p.tok_pos[t];
    const int* bt = L.block_table + (size_t)p.tok_seg[t] * p.max_blocks;
    const int first = (L.window > 0 && pos - L.window + 1 > 0) ? pos - L.window + 1 : 0;
    const int start = first & ~15;
    const int total = pos + 1 - start;
    int chunk = (total + splits - 1) / splits;
    chunk = (chunk + 15) & ~15;
    const int k_begin = start + split * chunk;
    int k_stop = k_begin + chunk;
    if (k_stop > pos + 1) k_stop = pos + 1;
    const bf16* qtok = p.q_buf + (size_t)t * p.H * HD + (size_t)kvh * G * HD;
    QFrag<HD> qf;
    load_q_cg<HD>(qf, g < G ? qtok + (size_t)g * HD : nullptr, g + 8 < G ? qtok + (size_t)(g + 8) * HD : nullptr, tg);
    const int lo[2] = {first, first};
    const int hi[2] = {g < G ? pos : -1, g + 8 < G ? pos : -1};
    RowState<HD> st;
    st.init();
    int pg = k_begin / p.page, in_pg = k_begin - pg * p.page;      // page and offset of the block, kept as counters
    for (int base = k_begin; base < k_stop; base += 16) {
      const bf16* kblk = L.cache + (size_t)bt[pg] * page_elems + ((size_t)kvh * p.page + in_pg) * HD;
      block16<HD, true>(st, qf, kblk, kblk + v_off, base, lo, hi, L.scale_log2, g, tg);
      in_pg += 16;
      if (in_pg == p.page) { in_pg = 0; ++pg; }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
      st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      if (row >= G) continue;
      float* dst = p.attn_partial + (((size_t)t * p.H + kvh * G + row) * splits + split) * ROW;
#pragma unroll
      for (int i = 0; i < Shape<HD>::NT; ++i) {
        dst[out_dim<HD>(i, 2 * tg)] = st.o[i][2 * r];
        dst[out_dim<HD>(i, 2 * tg + 1)] = st.o[i][2 * r + 1];
      }
      if (tg == 0) { dst[HD] = st.m[r]; dst[HD + 1] = st.l[r]; }
    }
  }
}

// One warp = one (token, head): merges the key slices in slice order; eight slices' loads at a time
__device__ __forceinline__ void step_combine(const FusedParams& p, int gw, int GW, int lane) {
  const int hd = p.hd, row = hd + 2, splits = p.splits;
  for (int item = gw; item < p.M * p.H; item += GW) {
    const float* src = p.attn_partial + (size_t)item * splits * row;
    float m = -INFINITY;
    for (int s = lane; s < splits; s += 32) m = fmaxf(m, __ldcg(src + (size_t)s * row + hd));
    m = warp_max(m);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float l = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 8) {
      float ms[8], ls[8], v[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool in = s0 + j < splits;
        const float* q = src + (size_t)(s0 + j) * row;
        ms[j] = in ? __ldcg(q + hd) : -INFINITY;
        ls[j] = in ? __ldcg(q + hd + 1) : 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) v[j][k] = (in && lane + 32 * k < hd) ? __ldcg(q + lane + 32 * k) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = (ms[j] == -INFINITY) ? 0.f : exp2f(ms[j] - m);
        l += ls[j] * f;
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[k] += v[j][k] * f;
      }
    }
    bf16* o = p.attn_out + (size_t)item * hd;       // item = t * H + h and the row is [H][hd]
    const float inv = 1.f / l;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int dd = lane + 32 * k;
      if (dd < hd) o[dd] = __float2bfloat16_rn(acc[k] * inv);
    }
  }
}

// act[tok][j] = silu(gate_j) * up_j from the parts of the gate/up product (times the token's 1/rms).
// One warp = one (token, 128 consecutive features); rows of the product are interleaved by 16
// (16 gate rows, the 16 up rows of the same features) or, if not, all gate rows then all up rows.
template <int BN>
__device__ __forceinline__ void step_swiglu(const FusedParams& p, const Ctl* ctl, const FusedLayer& L, int gw, int GW, int lane) {
  const float* ws = p.ws[2];
  const int mp = L.max_parts[2];
  const int groups = (p.f + 127) / 128;
  for (int item = gw; item < p.M * groups; item += GW) {
    const int tok = item / groups, j0 = (item - tok * groups) * 128 + 4 * lane;
    const float scale = row_scale(p, tok, L.eps2, lane);
    if (j0 >= p.f) continue;
    if (L.interleaved) {
      const int grow = (j0 >> 4) * 32 + (j0 & 15);          // gate row; the up row is 16 further
      const int t = grow / BM, r = grow - t * BM;
      const Parts q = parts_of(ws, mp, ctl, 2, t, BN);
      float4 g4 = parts_sum4(q, tok, r), u4 = parts_sum4(q, tok, r + 16);
      g4.x *= scale; g4.y *= scale; g4.z *= scale; g4.w *= scale;
      u4.x *= scale; u4.y *= scale; u4.z *= scale; u4.w *= scale;
      uint2 out;
      out.x = pack2_bf16(silu_mul(g4.x, u4.x), silu_mul(g4.y, u4.y));
      out.y = pack2_bf16(silu_mul(g4.z, u4.z), silu_mul(g4.w, u4.w));
      *(uint2*)(p.act + (size_t)tok * p.f + j0) = out;
    } else {
      for (int e = 0; e < 4 && j0 + e < p.f; ++e) {
        const int gr = j0 + e, ur = p.f + j0 + e;
        const int tg = gr / BM, tu = ur / BM;
        const float g = parts_sum1(parts_of(ws, mp, ctl, 2, tg, BN), tok, gr - tg * BM) * scale;
        const float u = parts_sum1(parts_of(ws, mp, ctl, 2, tu, BN), tok, ur - tu * BM) * scale;
        p.act[(size_t)tok * p.f + j0 + e] = __float2bfloat16_rn(silu_mul(g, u));
      }
    }
  }
}

// ------------------------------------------------------------------ the kernel
template <int BN>
__global__ void __launch_bounds__(FUSED_THREADS, 1) decode_fused_kernel(const __grid_constant__ FusedParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int X_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = W_TILE_BYTES + X_BYTES;
  constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = p.stages;
  Ctl* ctl = (Ctl*)(tiles + (size_t)S * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&ctl->full[s], 1 + X_LOADER_WARPS); mbar_init(&ctl->empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&ctl->acc_full[b], 1); mbar_init(&ctl->acc_empty[b], 4); }
    ctl->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_proxy();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_slot;

  if (warp == 0) {
    // ---------------- weight tiles, ahead of everything
    // (the three single-thread loops keep stage, phase, tile and k block as running counters:
    // a division by a run-time value is a chain of ~35 dependent instructions, which at one
    // warp's issue rate would pace the whole pipeline)
    if (lane == 0) {
      uint32_t i = 0;
      int s = 0;
      uint32_t ph = 0;                       // phase of the current use of stage s
      for (int l = 0; l < p.num_layers && !aborted(ctl); ++l) {
        const FusedLayer& L = p.layers[l];
        for (int gi = 0; gi < 4 && !aborted(ctl); ++gi) {
          Product pr; pr.set(L.n[gi], L.k[gi], G);
          const int u0 = share_begin(cta, pr.sh), u1 = share_begin(cta + 1, pr.sh);
          int t = u0 / pr.kbs, kb = u0 - t * pr.kbs;
          const CUtensorMap* wmap = &L.w[gi];
          for (int u = u0; u < u1; ++u, ++i) {
            if (!wait_bar(&ctl->empty[s], ph ^ 1, ctl, p.err, 11)) break;
            mbar_expect_tx(&ctl->full[s], W_TILE_BYTES);
            tma_load_2d(tiles + (size_t)s * STAGE_BYTES, wmap, &ctl->full[s], kb * BK, t * BM);
            if (++kb == pr.kbs) { kb = 0; ++t; }
            if (++s == S) { s = 0; ph ^= 1; }
          }
        }
      }
      // copies of stages that nothing consumed (only after a failure) are awaited before the
      // shared memory goes away
      if (aborted(ctl)) {
        const uint32_t from = i > (uint32_t)S ? i - S : 0;
        for (uint32_t j = from; j < i; ++j)
          for (uint32_t spin = 0; spin < (1u << 16); ++spin)
            if (mbar_try_wait(&ctl->full[j % S], (j / S) & 1)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BM, BN);
      uint32_t seg = 0;
      int s = 0;
      uint32_t ph = 0;
      for (int l = 0; l < p.num_layers && !aborted(ctl); ++l) {
        const FusedLayer& L = p.layers[l];
        for (int gi = 0; gi < 4 && !aborted(ctl); ++gi) {
          Product pr; pr.set(L.n[gi], L.k[gi], G);
          const int u0 = share_begin(cta, pr.sh), u1 = share_begin(cta + 1, pr.sh);
          int u = u0;
          int tile_end = (u0 / pr.kbs + 1) * pr.kbs;          // first unit of the next tile
          while (u < u1) {
            const int seg_end = tile_end < u1 ? tile_end : u1;
            const uint32_t buf = seg & 1;
            if (!wait_bar(&ctl->acc_empty[buf], ((seg >> 1) & 1) ^ 1, ctl, p.err, 14)) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * BN;
            bool ok = true;
            for (int uu = u; uu < seg_end; ++uu) {
              ok = wait_bar(&ctl->full[s], ph, ctl, p.err, 15);
              if (!ok) break;
              tc_fence_after();
              const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
              const uint64_t da = umma_desc(a_addr), db = umma_desc(a_addr + W_TILE_BYTES);
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk)
                umma_f16(d_tmem, da + 2 * kk, db + 2 * kk, idesc, (uu > u || kk > 0) ? 1u : 0u);
              umma_commit(&ctl->empty[s]);
              if (++s == S) { s = 0; ph ^= 1; }
            }
            if (!ok) break;
            umma_commit(&ctl->acc_full[buf]);
            ++seg;
            u = seg_end;
            tile_end += pr.kbs;
          }
        }
      }
    }
  } else if (warp >= 4) {
    // ---------------- workers
    const int wt = threadIdx.x - 128;            // 0..255
    const int ww = wt >> 5;                      // worker warp 0..7
    const int gw = cta * (FUSED_WORKERS / 32) + ww, GW = G * (FUSED_WORKERS / 32);
    unsigned round = 0;
    uint32_t seg = 0;
    int xs = 0;                                  // activation loaders: stage and phase of the next unit
    uint32_t xph = 0;
    // one step ends: what was written becomes visible to every CTA, all CTAs meet
    auto step_end = [&]() {
      __threadfence();
      worker_bar();
      if (wt == 0) {
        ++round;
        if (p.trace) p.trace[((size_t)round * 2) * G + cta] = global_ns();
        grid_barrier(p, ctl, round);
        if (p.trace) p.trace[((size_t)round * 2 + 1) * G + cta] = global_ns();
      }
      worker_bar();
    };
    // Worker warps 4..7 bring the activation tile of each unit into its stage: BN rows x 64 k of
    // the product's input, with plain loads (L2) and stores in the 128-byte swizzle the MMA expects.
    // TMA would do it in one instruction, but its queue is in order and holds the weight tiles
    // requested ahead, so a small tile needed now would wait behind 16 KB ones needed later.
    auto load_x = [&](const FusedLayer& L, int gi) {
      Product pr; pr.set(L.n[gi], L.k[gi], G);
      const int u0 = share_begin(cta, pr.sh), u1 = share_begin(cta + 1, pr.sh);
      const int K = L.k[gi];
      const bf16* x = gi == 1 ? p.attn_out : (gi == 3 ? p.act : p.x_norm);
      const int xt = wt - 128;                   // 0..127: one 16-byte chunk of a 16-row tile each
      const int r0 = xt >> 3, c = xt & 7;        // row (within 16) and chunk of the row
      int kb = u0 % pr.kbs;
      constexpr int UNR = 4;                     // units whose loads are in flight together
      for (int u = u0; u < u1; u += UNR) {
        uint4 v[UNR][BN / 16];
#pragma unroll
        for (int j = 0; j < UNR; ++j) {
          int kbj = kb + j;
          if (kbj >= pr.kbs) kbj -= pr.kbs;       // UNR <= kbs is not needed: one wrap at most when kbs >= UNR
          while (kbj >= pr.kbs) kbj -= pr.kbs;
          const int k0 = kbj * BK + c * 8;
#pragma unroll
          for (int q = 0; q < BN / 16; ++q)
            v[j][q] = (u + j < u1 && k0 < K) ? __ldcg((const uint4*)(x + (size_t)(r0 + 16 * q) * K + k0)) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < UNR; ++j) {
          if (u + j >= u1) break;
          int ok = 1;
          if (lane == 0) ok = wait_bar(&ctl->empty[xs], xph ^ 1, ctl, p.err, 13) ? 1 : 0;
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) return;
          uint8_t* xtile = tiles + (size_t)xs * STAGE_BYTES + W_TILE_BYTES;
#pragma unroll
          for (int q = 0; q < BN / 16; ++q) {
            const int r = r0 + 16 * q;
            *(uint4*)(xtile + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)) = v[j][q];
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->full[xs]);
          if (++xs == S) { xs = 0; xph ^= 1; }
        }
        kb += UNR;
        while (kb >= pr.kbs) kb -= pr.kbs;
      }
    };
    // drains this CTA's accumulators of one product into the workspace (worker warps 0..3)
    auto drain = [&](const FusedLayer& L, int gi) {
      if (ww >= 4) { load_x(L, gi); return; }
      Product pr; pr.set(L.n[gi], L.k[gi], G);
      const int u0 = share_begin(cta, pr.sh), u1 = share_begin(cta + 1, pr.sh);
      const int mp = L.max_parts[gi];
      int u = u0;
      while (u < u1) {
        const int t = u / pr.kbs;
        const int seg_end = (t + 1) * pr.kbs < u1 ? (t + 1) * pr.kbs : u1;
        const uint32_t buf = seg & 1;
        int ok = 1;
        if (lane == 0) ok = wait_bar(&ctl->acc_full[buf], (seg >> 1) & 1, ctl, p.err, 16) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) {
          tc_fence_after();
          const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(ww * 32) << 16);
          float* dst = p.ws[gi] + (((size_t)t * mp + (cta - pr.first_cta(t))) * BN) * BM + ww * 32 + lane;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(taddr + c0, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c0 + j < p.M) dst[(size_t)(c0 + j) * BM] = __uint_as_float(r[j]);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
        }
        ++seg;
        u = seg_end;
      }
    };

    if (wt == 0 && p.trace) p.trace[cta] = global_ns();
    step_add_prenorm<BN>(p, ctl, nullptr, 0, 0, p.layers[0].norm1, gw, GW, lane);
    step_end();
    for (int l = 0; l < p.num_layers; ++l) {
      const FusedLayer& L = p.layers[l];
      // parts of every tile of this layer's products (read from the next step on; the barrier
      // inside step_end lies between)
      {
        int off = 0;
        for (int gi = 0; gi < 4; ++gi) {
          Product pr; pr.set(L.n[gi], L.k[gi], G);
          if (wt == 0) ctl->part_off[gi] = off;
          for (int t = wt; t < pr.tiles; t += FUSED_WORKERS) ctl->part_count[off + t] = (uint8_t)(pr.last_cta(t) - pr.first_cta(t) + 1);
          off += pr.tiles;
        }
      }
      // every lane of a warp takes the same branch: the steps use warp-wide operations
      if (!__any_sync(0xffffffffu, aborted(ctl))) drain(L, 0);
      step_end();
      if (!__any_sync(0xffffffffu, aborted(ctl))) step_rope<BN>(p, ctl, L, gw, GW, lane);
      step_end();
      if (!__any_sync(0xffffffffu, aborted(ctl))) {
        switch (p.hd) {
          case 16: step_attention<16>(p, L, gw, GW, lane); break;
          case 32: step_attention<32>(p, L, gw, GW, lane); break;
          case 48: step_attention<48>(p, L, gw, GW, lane); break;
          case 64: step_attention<64>(p, L, gw, GW, lane); break;
          case 80: step_attention<80>(p, L, gw, GW, lane); break;
          case 96: step_attention<96>(p, L, gw, GW, lane); break;
          case 112: step_attention<112>(p, L, gw, GW, lane); break;
          default: step_attention<128>(p, L, gw, GW, lane); break;
        }
      }
      step_end();
      if (!__any_sync(0xffffffffu, aborted(ctl))) step_combine(p, gw, GW, lane);
      step_end();
      if (!__any_sync(0xffffffffu, aborted(ctl))) drain(L, 1);
      step_end();
      if (!__any_sync(0xffffffffu, aborted(ctl))) step_add_prenorm<BN>(p, ctl, p.ws[1], L.max_parts[1], 1, L.norm2, gw, GW, lane);
      step_end();
      if (!__any_sync(0xffffffffu, aborted(ctl))) drain(L, 2);
      step_end();
      if (!__any_sync(0xffffffffu, aborted(ctl))) step_swiglu<BN>(p, ctl, L, gw, GW, lane);
      step_end();
      if (!__any_sync(0xffffffffu, aborted(ctl))) drain(L, 3);
      step_end();
      const bool last = l + 1 == p.num_layers;
      if (!__any_sync(0xffffffffu, aborted(ctl)))
        step_add_prenorm<BN>(p, ctl, p.ws[3], L.max_parts[3], 3, last ? p.final_norm : p.layers[l + 1].norm1, gw, GW, lane);
      step_end();
      if (last && !__any_sync(0xffffffffu, aborted(ctl))) step_final_norm(p, p.final_norm, p.final_eps, gw, GW, lane);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------ host side
long long* g_trace = nullptr;
int g_sms = 0;
int sm_count() {
  if (g_sms <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_sms <= 0) g_sms = 148;
  }
  return g_sms;
}

int max_parts_of(int n, int k, int G) {
  const int tiles = (n + BM - 1) / BM, kbs = (k + BK - 1) / BK;
  const Share sh = make_share(tiles * kbs, G);
  int mp = 1;
  for (int t = 0; t < tiles; ++t) {
    const int c = share_owner((t + 1) * kbs - 1, sh) - share_owner(t * kbs, sh) + 1;
    if (c > mp) mp = c;
  }
  return mp;
}

template <int BN>
int launch_fused(const FusedParams& p, cudaStream_t st) {
  constexpr int STAGE_BYTES = W_TILE_BYTES + BN * BK * 2;
  static int stages = 0;
  static int smem = 0;
  if (!stages) {
    int dev = 0, max_smem = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    int s = (max_smem - 1024 - (int)sizeof(Ctl) - 64) / STAGE_BYTES;
    if (s > FUSED_MAX_STAGES) s = FUSED_MAX_STAGES;
    if (s < 2) return QV_ERR_TOO_LARGE;
    const int bytes = 1024 + s * STAGE_BYTES + (int)sizeof(Ctl) + 64;
    cudaError_t e = cudaFuncSetAttribute(decode_fused_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return (int)e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_fused_kernel<BN>, FUSED_THREADS, bytes);
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) return QV_ERR_TOO_LARGE;
    stages = s;
    smem = bytes;
  }
  FusedParams q = p;
  q.stages = stages;
  q.trace = g_trace;
  cudaError_t e = cudaMemsetAsync(p.barrier, 0, sizeof(unsigned), st);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(sm_count());
  cfg.blockDim = dim3(FUSED_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;      // all CTAs resident at once: they meet at barriers
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, decode_fused_kernel<BN>, q);
}

}  // namespace

// Profiling aid: with a device buffer of 64-bit words set here,
// later launches record when each CTA reached and left each step's barrier (%globaltimer, ns):
// [step][reached, left][CTA], step 0 being the start ((10 * layers + 2) * 2 * grid words).  Null: off.
extern "C" void qv_fused_set_trace(long long* buf) { g_trace = buf; }

// Sizes of the device records, for the caller's buffers.
extern "C" int qv_fused_layer_bytes() { return (int)sizeof(FusedLayer); }
extern "C" int qv_fused_grid() { return sm_count(); }

// Floats of partial-sum workspace that product (n rows, k long) needs with BN token columns.
extern "C" long long qv_fused_workspace_floats(int n, int k, int BN) {
  const int tiles = (n + BM - 1) / BM;
  return (long long)tiles * max_parts_of(n, k, sm_count()) * BN * BM;
}

// Fills one FusedLayer record (host memory, to be copied to the device by the caller).
// Refuses matrices that TMA cannot describe (k not a multiple of 8, unaligned base).
extern "C" int qv_fused_fill_layer(void* record, const FusedHostLayer* h) {
  FusedLayer L;
  memset(&L, 0, sizeof(L));
  const int G = sm_count();
  int total_tiles = 0;
  for (int i = 0; i < 4; ++i) {
    const int n = (int)h->n[i], k = (int)h->k[i];
    if (n <= 0 || k < 8 || (k & 7) || ((uintptr_t)h->w[i] & 15)) return QV_ERR_UNSUPPORTED;
    if (!make_map(&L.w[i], h->w[i], n, k, k, BM)) return QV_ERR_UNSUPPORTED;
    L.n[i] = n; L.k[i] = k;
    total_tiles += (n + BM - 1) / BM;
    L.max_parts[i] = max_parts_of(n, k, G);
  }
  if (total_tiles > FUSED_MAX_TILES) return QV_ERR_TOO_LARGE;
  L.norm1 = h->norm1; L.norm2 = h->norm2;
  L.cache = (bf16*)h->cache; L.block_table = h->block_table;
  L.eps1 = (float)h->eps1; L.eps2 = (float)h->eps2;
  L.window = (int)h->window;
  if (h->rot < 0 || (h->rot & 1) || (h->rope && h->rope_rows <= 0)) return QV_ERR_UNSUPPORTED;
  L.rope = (const float2*)h->rope; L.rot = (int)h->rot; L.rope_rows = (int)h->rope_rows;
  L.interleaved = h->interleaved ? 1 : 0;
  if (L.interleaved ? (h->n[2] & 31) != 0 : (h->n[2] & 1) != 0) return QV_ERR_UNSUPPORTED;
  L.scale_log2 = (float)(h->scale * 1.4426950408889634);
  memcpy(record, &L, sizeof(L));
  return 0;
}

// Runs all layers for M <= BN tokens.  resid holds the embedded tokens on entry and the residual
// stream after the last layer on return; x_norm then holds the final norm's output.
extern "C" int qv_fused_decode(const FusedHostArgs* a, void* stream) {
  const int M = (int)a->M, BN = (int)a->BN, hd = (int)a->hd, H = (int)a->H, Hkv = (int)a->Hkv;
  if (M <= 0 || a->num_layers <= 0) return 0;
  if (M > BN || (BN != 16 && BN != 32 && BN != 64)) return QV_ERR_UNSUPPORTED;
  if (hd < 16 || hd > 128 || (hd & 15) || Hkv <= 0 || H % Hkv || H / Hkv > 16) return QV_ERR_UNSUPPORTED;
  if ((a->d & 7) || (a->d & 3) || (a->f & 7) || (a->page & 15) || a->splits < 1) return QV_ERR_UNSUPPORTED;
  FusedParams p;
  memset(&p, 0, sizeof(p));
  p.layers = (const FusedLayer*)a->layers;
  p.final_norm = a->final_norm;
  p.resid = a->resid;
  p.x_norm = (bf16*)a->x_norm; p.q_buf = (bf16*)a->q_buf; p.attn_out = (bf16*)a->attn_out; p.act = (bf16*)a->act;
  for (int i = 0; i < 4; ++i) p.ws[i] = a->ws[i];
  p.attn_partial = a->attn_partial;
  p.ssq = a->ssq;
  p.tok_pos = a->tok_pos; p.tok_seg = a->tok_seg;
  p.barrier = a->barrier; p.err = a->err;
  p.num_layers = (int)a->num_layers; p.M = M; p.d = (int)a->d; p.H = H; p.Hkv = Hkv; p.hd = hd;
  p.f = (int)a->f; p.page = (int)a->page; p.max_blocks = (int)a->max_blocks; p.splits = (int)a->splits;
  p.final_eps = (float)a->final_eps;
  cudaStream_t st = (cudaStream_t)stream;
  if (BN == 16) return launch_fused<16>(p, st);
  if (BN == 32) return launch_fused<32>(p, st);
  return launch_fused<64>(p, st);
}
