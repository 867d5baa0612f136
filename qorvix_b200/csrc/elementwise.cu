// Memory-bound kernels of the step: embedding gather, (residual add +) RMSNorm (+ row
// gather), rotary encoding fused with the paged key/value write, SwiGLU, casts.
// Formulas follow the reference's CPU ops (runtime/src/ops.cpp:8-13 rmsnorm, :96-100 swiglu,
// :127-148 split-half rope) and its CUDA twins (cuda/src/cuda_backend.cu:231-340), rebuilt
// for batches of tokens, a float32 residual stream and a paged cache.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] as float32 (the residual stream is float32).
template <typename TW>
__global__ void embed_kernel(float* __restrict__ out, const TW* __restrict__ table,
                             const int* __restrict__ ids, int d, int vocab) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;   // ids are validated on the host; never read out of bounds
  const TW* row = table + (size_t)id * d;
  float* o = out + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f(row[i]);
}

extern "C" int qv_embed(float* out, const void* table, const int* ids, int T, int d, int vocab,
                        int table_dt, void* stream) {
  if (T <= 0) return 0;
  QV_DISPATCH_DT(table_dt, TW,
                 return qv_launch(embed_kernel<TW>, dim3(T), dim3(256), 0, (cudaStream_t)stream, out, (const TW*)table, ids, d, vocab));
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- add + rmsnorm (+ gather)
// row r reads source row s = row_idx ? row_idx[r] : r.
//   x = residual[s] + (delta ? delta[s] : 0)        (float32 sum)
//   if write_residual: residual[s] = x              (only without row_idx)
//   out[r] = (x * rsqrt(mean(x^2) + eps)) * w
// One block per row; the row is staged in shared memory so it is read once.
template <typename TD> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *(const float4*)p; }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 v = *(const uint2*)p;
    const __nv_bfloat162 a = *(const __nv_bfloat162*)&v.x, b = *(const __nv_bfloat162*)&v.y;
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
};
__device__ __forceinline__ void store4(float* p, float4 v) { *(float4*)p = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u; u.x = *(uint32_t*)&a; u.y = *(uint32_t*)&b;
  *(uint2*)p = u;
}

// VEC: rows are read four elements at a time, all loads of a thread issued before any is used
// (d a multiple of 4, at most 4 * 4 * blockDim elements); else one element at a time.
template <typename TD, typename TO, bool VEC>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(TO* __restrict__ out, float* __restrict__ residual,
                                   const TD* __restrict__ delta, const float* __restrict__ w,
                                   const int* __restrict__ row_idx, int d, float eps,
                                   int write_residual) {
  extern __shared__ float smem[];
  pdl_wait();
  pdl_launch_dependents();
  float* xs = smem;            // d floats
  float* red = VEC ? smem : smem + d;       // 33 floats
  const int r = blockIdx.x;
  const int s = row_idx ? row_idx[r] : r;
  float* res = residual + (size_t)s * d;
  const TD* dl = delta ? delta + (size_t)s * d : nullptr;
  TO* o = out + (size_t)r * d;
  float ss = 0.f;
  if constexpr (VEC) {
    constexpr int MAXV = 4;
    float4 x[MAXV];
    const int nvec = d >> 2;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * 256;
      x[k] = i < nvec ? *(const float4*)(res + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (dl) {
#pragma unroll
      for (int k = 0; k < MAXV; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < nvec) {
          const float4 dv = Vec4<TD>::load(dl + 4 * i);
          x[k].x += dv.x; x[k].y += dv.y; x[k].z += dv.z; x[k].w += dv.w;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < nvec) {
        if (write_residual) *(float4*)(res + 4 * i) = x[k];
        ss += x[k].x * x[k].x + x[k].y * x[k].y + x[k].z * x[k].z + x[k].w * x[k].w;
      }
    }
    const float total = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(total / (float)d + eps);
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < nvec) {
        const float4 wv = *(const float4*)(w + 4 * i);
        store4(o + 4 * i, make_float4(x[k].x * scale * wv.x, x[k].y * scale * wv.y, x[k].z * scale * wv.z, x[k].w * scale * wv.w));
      }
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      float x = res[i];
      if (dl) x += to_f(dl[i]);
      xs[i] = x;
      if (write_residual) res[i] = x;
      ss += x * x;
    }
    const float total = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(total / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_f<TO>(xs[i] * scale * w[i]);
  }
}

extern "C" int qv_add_rmsnorm(void* out, float* residual, const void* delta, const float* w,
                              const int* row_idx, int rows, int d, float eps, int write_residual,
                              int delta_dt, int out_dt, void* stream) {
  if (rows <= 0) return 0;
  const size_t smem = (size_t)(d + 33) * sizeof(float);
  if (smem > 200 * 1024) return QV_ERR_TOO_LARGE;
  if (row_idx && write_residual) return QV_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  int rc = 0;
  // the vector path keeps the row in registers: d a multiple of 4, at most 4096 elements, rows 16-byte aligned
  const bool vec = (d % 4 == 0) && d <= 4 * 4 * 256 && (((uintptr_t)out | (uintptr_t)residual | (uintptr_t)delta | (uintptr_t)w) & 15) == 0;
#define LAUNCH_NORM(TD, TO)                                                                          \
  do {                                                                                               \
    if (vec) {                                                                                       \
      rc = qv_launch(add_rmsnorm_kernel<TD, TO, true>, dim3(rows), dim3(256), 48 * sizeof(float), st, \
          (TO*)out, residual, (const TD*)delta, w, row_idx, d, eps, write_residual);                 \
    } else {                                                                                         \
      if (smem > 48 * 1024)                                                                          \
        cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO, false>,                                      \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                \
      rc = qv_launch(add_rmsnorm_kernel<TD, TO, false>, dim3(rows), dim3(256), smem, st, (TO*)out, residual, \
                                                 (const TD*)delta, w, row_idx, d, eps, write_residual); \
    }                                                                                                \
  } while (0)
  if (delta_dt == QV_DT_F32 && out_dt == QV_DT_F32) LAUNCH_NORM(float, float);
  else if (delta_dt == QV_DT_BF16 && out_dt == QV_DT_BF16) LAUNCH_NORM(bf16, bf16);
  else if (delta_dt == QV_DT_F32 && out_dt == QV_DT_BF16) LAUNCH_NORM(float, bf16);
  else if (delta_dt == QV_DT_BF16 && out_dt == QV_DT_F32) LAUNCH_NORM(bf16, float);
  else return QV_ERR_UNSUPPORTED;
#undef LAUNCH_NORM
  return rc;
}

// ---------------------------------------------------------------- rotary + paged KV write
// qkv[t] = [q: H*hd | k: Hkv*hd | v: Hkv*hd] in the compute dtype (row stride `ld`).
// For token t at position p (table row p holds cos/sin of p*inv_freq[i], i < rot/2):
//   q heads and k heads: pairs (i, i + rot/2) of the first `rot` dims are rotated
//   (split-half), the other dims pass through.  q is rewritten in place; the rotated k and
//   the plain v go to the cache slot of (request, position):
//   page = block_table[seg, p / page], cache[page][0|1][kv head][p % page][:]
// If `cache` is null only q and k are rotated in place (k is then written back to qkv).
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int ld, T* __restrict__ cache,
                                     const float2* __restrict__ cos_sin, int table_rows,
                                     const int* __restrict__ tok_pos, const int* __restrict__ tok_seg,
                                     const int* __restrict__ block_table, int max_blocks, int H,
                                     int Hkv, int hd, int rot, int page) {
  // grid (token, groups of 8 head slots), one warp per slot: slots 0..H-1 are q heads,
  // H..H+Hkv-1 k heads, H+Hkv..H+2Hkv-1 v heads
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int head = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (head >= H + 2 * Hkv) return;
  const int lane = threadIdx.x & 31;
  const int pos = tok_pos[t];
  T* row = qkv + (size_t)t * ld;
  const int half = rot >> 1;
  const float2* cs = cos_sin + (size_t)(pos < table_rows ? pos : table_rows - 1) * half;
  T* kdst = nullptr;
  T* vdst = nullptr;
  if (cache) {
    const int pg = block_table[(size_t)tok_seg[t] * max_blocks + pos / page];
    const size_t page_elems = (size_t)2 * Hkv * page * hd;
    kdst = cache + (size_t)pg * page_elems + (size_t)(pos % page) * hd;
    vdst = kdst + (size_t)Hkv * page * hd;
  }
  if (head < H + Hkv) {
    T* v = row + (size_t)head * hd;
    const bool to_cache = head >= H && cache;
    T* dst = to_cache ? kdst + (size_t)(head - H) * page * hd : v;
    if (sizeof(T) == 2 && (half & 1) == 0 && (((uintptr_t)v | (uintptr_t)dst) & 3) == 0) {
      // bfloat16: two neighbouring pairs per lane, 4-byte loads and stores
      for (int i = 2 * lane; i < half; i += 64) {
        const __nv_bfloat162 a2 = *(const __nv_bfloat162*)((const bf16*)v + i);
        const __nv_bfloat162 b2 = *(const __nv_bfloat162*)((const bf16*)v + i + half);
        const float2 c0 = cs[i], c1 = cs[i + 1];
        const float a0 = __low2float(a2), a1 = __high2float(a2), b0 = __low2float(b2), b1 = __high2float(b2);
        *(__nv_bfloat162*)((bf16*)dst + i) = __floats2bfloat162_rn(a0 * c0.x - b0 * c0.y, a1 * c1.x - b1 * c1.y);
        *(__nv_bfloat162*)((bf16*)dst + i + half) = __floats2bfloat162_rn(a0 * c0.y + b0 * c0.x, a1 * c1.y + b1 * c1.x);
      }
    } else {
      for (int i = lane; i < half; i += 32) {
        const float a = to_f(v[i]), b = to_f(v[i + half]);
        const float2 c = cs[i];
        dst[i] = from_f<T>(a * c.x - b * c.y);
        dst[i + half] = from_f<T>(a * c.y + b * c.x);
      }
    }
    if (to_cache)      // dims beyond the rotated ones pass through
      for (int i = rot + lane; i < hd; i += 32) dst[i] = v[i];
  } else if (cache) {
    const int vh = head - H - Hkv;
    const T* v = row + (size_t)head * hd;
    T* dst = vdst + (size_t)vh * page * hd;
    if (sizeof(T) == 2 && (hd & 7) == 0 && (((uintptr_t)v | (uintptr_t)dst) & 15) == 0) {
      for (int i = 8 * lane; i < hd; i += 256) *(uint4*)((bf16*)dst + i) = *(const uint4*)((const bf16*)v + i);
    } else {
      for (int i = lane; i < hd; i += 32) dst[i] = v[i];
    }
  }
}

extern "C" int qv_rope_kv_write(void* qkv, int ld, void* cache, const float* cos_sin, int table_rows,
                                const int* tok_pos, const int* tok_seg, const int* block_table,
                                int max_blocks, int T, int H, int Hkv, int hd, int rot, int page,
                                int dt, void* stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > hd || (rot & 1)) return QV_ERR_UNSUPPORTED;
  if ((H + 2 * Hkv + 7) / 8 > 65535) return QV_ERR_TOO_LARGE;
  QV_DISPATCH_DT(dt, TT,
                 return qv_launch(rope_kv_write_kernel<TT>, dim3(T, (H + 2 * Hkv + 7) / 8), dim3(256), 0, (cudaStream_t)stream,
                     (TT*)qkv, ld, (TT*)cache, (const float2*)cos_sin, table_rows, tok_pos, tok_seg,
                     block_table, max_blocks, H, Hkv, hd, rot, page));
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- swiglu
// out[t, i] = gate/(1+exp(-gate)) * up, with gu[t] (row stride 2f) either [gate: f | up: f] or, when
// `interleaved`, groups of 32 columns holding 16 gate values and then the 16 up values of the same
// features (the layout the fused tensor-core epilogue uses; f a multiple of 16).
template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gu, size_t n, int f, int interleaved) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / f;
    const int i = (int)(idx - t * f);
    const int gi = interleaved ? ((i >> 4) << 5) + (i & 15) : i;
    const int ui = interleaved ? gi + 16 : f + i;
    const float g = to_f(gu[t * 2 * f + gi]);
    const float u = to_f(gu[t * 2 * f + ui]);
    out[idx] = from_f<T>(g / (1.0f + expf(-g)) * u);
  }
}

extern "C" int qv_swiglu(void* out, const void* gu, int T, int f, int interleaved, int dt, void* stream) {
  const size_t n = (size_t)T * f;
  if (n == 0) return 0;
  if (interleaved && (f & 15)) return QV_ERR_UNSUPPORTED;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  QV_DISPATCH_DT(dt, TT, return qv_launch(swiglu_kernel<TT>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (TT*)out, (const TT*)gu, n, f, interleaved));
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- casts
template <typename TI, typename TO>
__global__ void cast_kernel(TO* __restrict__ out, const TI* __restrict__ in, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f<TO>(to_f(in[i]));
}

extern "C" int qv_cast(void* out, const void* in, long long n, int in_dt, int out_dt, void* stream) {
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dt == QV_DT_F32 && out_dt == QV_DT_BF16) cast_kernel<float, bf16><<<blocks, 256, 0, st>>>((bf16*)out, (const float*)in, (size_t)n);
  else if (in_dt == QV_DT_BF16 && out_dt == QV_DT_F32) cast_kernel<bf16, float><<<blocks, 256, 0, st>>>((float*)out, (const bf16*)in, (size_t)n);
  else return QV_ERR_UNSUPPORTED;
  return qv_launch_status();
}

// out[r, c] = in[r, c] for matrices whose rows are contiguous but may lie any stride apart, with a
// change of type on the way if asked: what makes an aligned, dense copy of a column slice of a wider
// buffer, or of float32 rows for a kernel that takes bfloat16.
template <typename FROM, typename TO>
__global__ void cast_rows_kernel(TO* __restrict__ out, long long ld_out, const FROM* __restrict__ in, long long ld_in, int rows, int cols) {
  const size_t n = (size_t)rows * cols;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / cols, c = i - r * cols;
    out[r * ld_out + c] = from_f<TO>(to_f(in[r * ld_in + c]));
  }
}

extern "C" int qv_cast_rows(void* out, long long ld_out, const void* in, long long ld_in, int rows, int cols, int in_dt, int out_dt, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const size_t n = (size_t)rows * cols;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  cudaStream_t st = (cudaStream_t)stream;
#define QV_CAST_ROWS(FROM, TO) cast_rows_kernel<FROM, TO><<<blocks, 256, 0, st>>>((TO*)out, ld_out, (const FROM*)in, ld_in, rows, cols)
  if (in_dt == QV_DT_F32 && out_dt == QV_DT_BF16) QV_CAST_ROWS(float, bf16);
  else if (in_dt == QV_DT_BF16 && out_dt == QV_DT_F32) QV_CAST_ROWS(bf16, float);
  else if (in_dt == QV_DT_F32 && out_dt == QV_DT_F32) QV_CAST_ROWS(float, float);
  else if (in_dt == QV_DT_BF16 && out_dt == QV_DT_BF16) QV_CAST_ROWS(bf16, bf16);
  else return QV_ERR_UNSUPPORTED;
#undef QV_CAST_ROWS
  return qv_launch_status();
}

extern "C" const char* qv_error_string(int code) {
  if (code == QV_ERR_UNSUPPORTED) return "size or dtype not supported by this kernel";
  if (code == QV_ERR_TOO_LARGE) return "size exceeds what this kernel can hold on chip";
  return cudaGetErrorString((cudaError_t)code);
}
