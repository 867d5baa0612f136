// Causal grouped-query attention over the paged cache, one warp per (token, query head).
// It serves every kind of step (a prompt portion, a single decoded token, any mix) with
// the same arithmetic, in float32 whatever the storage type, and takes any head size.
// It is the attention of the true 32-bit path and the reference for the tensor-core kernels.
//
// Formula (reference: runtime/src/text_model.cpp:83-114; its CUDA twin keeps all scores in
// shared memory and runs the softmax on one thread, cuda/src/cuda_backend.cu:347-395):
//   kv head = h / (H / Hkv);  s_t = (q . K_t) * scale for lo <= t <= pos;
//   p = softmax(s);  out = sum_t p_t V_t          lo = 0, or pos - window + 1 with a window.
//
// Keys are visited in blocks of 32 aligned to absolute positions (0-31, 32-63, ...), with a
// running maximum and sum, so the result for a position depends on that position and the
// cache contents only: not on how the prompt was cut, nor on the rest of the batch.
#include "common.cuh"

#define MAX_HD 512

template <typename T>
__global__ void __launch_bounds__(128) attention_generic_kernel(
    T* __restrict__ out, int ld_out, const T* __restrict__ q, int ld_q, const T* __restrict__ cache,
    const int* __restrict__ tok_pos, const int* __restrict__ tok_seg,
    const int* __restrict__ block_table, int max_blocks, int H, int Hkv, int hd, int page, int window,
    float scale) {
  extern __shared__ float qs_all[];              // 4 warps x hd floats
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x * 4 + warp;
  const int t = blockIdx.y;
  if (h >= H) return;                            // whole warp leaves together
  float* qs = qs_all + (size_t)warp * hd;
  const T* qrow = q + (size_t)t * ld_q + (size_t)h * hd;
  for (int i = lane; i < hd; i += 32) qs[i] = to_f(qrow[i]);
  __syncwarp();

  const int pos = tok_pos[t];
  const int* bt = block_table + (size_t)tok_seg[t] * max_blocks;
  const int kvh = h / (H / Hkv);
  const int lo = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
  const size_t page_elems = (size_t)2 * Hkv * page * hd;
  const size_t v_off = (size_t)Hkv * page * hd;
  const size_t head_off = (size_t)kvh * page * hd;

  constexpr int NREG = MAX_HD / 32;
  float o[NREG];
#pragma unroll
  for (int j = 0; j < NREG; ++j) o[j] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int kb = (lo >> 5) << 5; kb <= pos; kb += 32) {
    const int tk = kb + lane;
    const bool valid = tk >= lo && tk <= pos;
    size_t base = 0;
    float s = -INFINITY;
    if (valid) {
      base = (size_t)bt[tk / page] * page_elems + head_off + (size_t)(tk % page) * hd;
      const T* kp = cache + base;
      float dot = 0.f;
      for (int i = 0; i < hd; ++i) dot = fmaf(qs[i], to_f(kp[i]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));   // finite: the block holds at least one valid key
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);          // exp(-inf) = 0 for the first block
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int j = 0; j < NREG; ++j) o[j] *= corr;
    const int nk = pos - kb + 1 < 32 ? pos - kb + 1 : 32;
    for (int j = 0; j < nk; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const size_t bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
      if (pj == 0.f) continue;                   // masked (before the window) or underflowed: adds nothing
      const T* vp = cache + bj + v_off;
#pragma unroll
      for (int r = 0; r < NREG; ++r) {
        const int i = lane + 32 * r;
        if (i < hd) o[r] = fmaf(pj, to_f(vp[i]), o[r]);
      }
    }
    m = m_new;
  }
  T* orow = out + (size_t)t * ld_out + (size_t)h * hd;
  const float inv = 1.0f / l;
#pragma unroll
  for (int r = 0; r < NREG; ++r) {
    const int i = lane + 32 * r;
    if (i < hd) orow[i] = from_f<T>(o[r] * inv);
  }
}

extern "C" int qv_attention_generic(void* out, int ld_out, const void* q, int ld_q, const void* cache,
                                    const int* tok_pos, const int* tok_seg, const int* block_table,
                                    int max_blocks, int T, int H, int Hkv, int hd, int page,
                                    int window, float scale, int dt, void* stream) {
  if (T <= 0) return 0;
  if (hd > MAX_HD || hd <= 0 || Hkv <= 0 || H % Hkv) return QV_ERR_UNSUPPORTED;
  if (T > 65535 * 32) return QV_ERR_TOO_LARGE;
  dim3 grid((H + 3) / 4, T);
  if (grid.y > 65535) {
    // split over several launches; rows are independent
    int done = 0;
    while (done < T) {
      const int n = T - done < 65535 ? T - done : 65535;
      const size_t esz = dt == QV_DT_F32 ? 4 : 2;
      int rc = qv_attention_generic((char*)out + (size_t)done * ld_out * esz, ld_out,
                                    (const char*)q + (size_t)done * ld_q * esz, ld_q, cache,
                                    tok_pos + done, tok_seg + done, block_table, max_blocks, n, H, Hkv,
                                    hd, page, window, scale, dt, stream);
      if (rc) return rc;
      done += n;
    }
    return 0;
  }
  const size_t smem = (size_t)4 * hd * sizeof(float);
  QV_DISPATCH_DT(dt, TT,
                 attention_generic_kernel<TT><<<grid, 128, smem, (cudaStream_t)stream>>>(
                     (TT*)out, ld_out, (const TT*)q, ld_q, (const TT*)cache, tok_pos, tok_seg,
                     block_table, max_blocks, H, Hkv, hd, page, window, scale));
  return qv_launch_status();
}
