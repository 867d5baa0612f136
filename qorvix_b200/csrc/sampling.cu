// On-device sampling over float32 logits [rows, vocab]: greedy argmax, and the reference's
// sampler (runtime/src/sampler.cpp:13-101) in its order of operations:
//   penalties over the recent tokens -> greedy if temperature <= 0 -> logits / temperature ->
//   softmax -> top-k -> top-p (shortest prefix of the sorted list whose cumulative probability
//   reaches p, probabilities not renormalised) -> min-p (drop p < min_p * p_max) -> draw.
// One block per row.  Instead of sorting the vocabulary, every token gets a unique 64-bit key
// (order-preserving bits of its scaled logit, then lowest id first among equals); top-k and
// top-p become thresholds on that key found by radix descent (8 passes of 8 bits each).
// Probabilities are held as 2^40 fixed-point integers, so every sum is exact and the result
// does not depend on the order in which threads add: the same row and the same uniform number
// always give the same token, whatever else is in the batch.
// The draw walks the survivors in id order (the reference walks them in sorted order; the
// distribution is the same, the token for a given random number is not).
#include "common.cuh"

#define SAMPLE_THREADS 1024
typedef unsigned long long u64;

__device__ __forceinline__ unsigned ordered_bits(float f) {
  unsigned b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ u64 unique_key(float x, int i) {
  return ((u64)ordered_bits(x) << 32) | (u64)(0xFFFFFFFFu - (unsigned)i);
}
__device__ __forceinline__ u64 fixed_weight(float x, float xmax) {
  return (u64)(expf(x - xmax) * 1099511627776.0f);   // 2^40; exp(0) = 1 maps to 2^40 exactly
}

// ---------------------------------------------------------------- argmax (first maximum wins)
__global__ void argmax_kernel(int* __restrict__ out, const float* __restrict__ logits, int V, long long ld) {
  pdl_wait();
  pdl_launch_dependents();
  const float* row = logits + (size_t)blockIdx.x * ld;
  float best = -INFINITY;
  int besti = 0x7fffffff;
  if ((((uintptr_t)row) & 15) == 0) {
    // four independent 16-byte loads in flight per thread
    const int nvec = V >> 2;
    const float4* row4 = (const float4*)row;
    for (int i0 = threadIdx.x; i0 < nvec; i0 += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = i0 + k * blockDim.x;
        v[k] = i < nvec ? row4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = 4 * (i0 + k * blockDim.x);
        const float e[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (e[j] > best || (e[j] == best && i + j < besti)) { best = e[j]; besti = i + j; }
      }
    }
    for (int i = (nvec << 2) + threadIdx.x; i < V; i += blockDim.x) {
      const float v = row[i];
      if (v > best || (v == best && i < besti)) { best = v; besti = i; }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = row[i];
      if (v > best || (v == best && i < besti)) { best = v; besti = i; }
    }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = besti; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    besti = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = besti == 0x7fffffff ? 0 : besti;
  }
}

extern "C" int qv_argmax(int* out, const float* logits, int rows, int V, long long ld, void* stream) {
  if (rows <= 0) return 0;
  return qv_launch(argmax_kernel, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, out, logits, V, ld);
}

// ---------------------------------------------------------------- sampler
struct SampleShared {
  unsigned count[256];
  u64 mass[256];
  u64 red[33];
  float fred[33];
  u64 bcast[4];
};

__device__ __forceinline__ u64 block_sum_u64(u64 v, SampleShared& sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh.red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    u64 t = threadIdx.x < (blockDim.x >> 5) ? sh.red[threadIdx.x] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) sh.red[32] = t;
  }
  __syncthreads();
  return sh.red[32];
}

// Radix descent over the unique keys >= floor_key.  by_mass == 0: the key of rank `target`
// (1 = largest) by count.  by_mass == 1: the largest key K with mass{key >= K} >= target.
// Returns floor_key when the whole set falls short of the target.
__device__ u64 radix_threshold(const float* row, int V, float inv_t, float xmax, u64 floor_key,
                               u64 target, int by_mass, SampleShared& sh) {
  u64 prefix = 0;        // bits decided so far (high part)
  u64 acc = 0;           // count or mass of keys strictly above the current prefix range
  for (int shift = 56; shift >= 0; shift -= 8) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) { sh.count[b] = 0; sh.mass[b] = 0; }
    __syncthreads();
    const u64 hi_mask = shift == 56 ? 0 : (~0ull << (shift + 8));
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = row[i] * inv_t;
      const u64 key = unique_key(x, i);
      if (key < floor_key || (key & hi_mask) != prefix) continue;
      const int b = (int)((key >> shift) & 0xff);
      if (by_mass) atomicAdd(&sh.mass[b], fixed_weight(x, xmax));
      else atomicAdd(&sh.count[b], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int chosen = -1;
      u64 a = acc;
      for (int b = 255; b >= 0; --b) {
        const u64 w = by_mass ? sh.mass[b] : (u64)sh.count[b];
        if (a + w >= target) { chosen = b; break; }
        a += w;
      }
      sh.bcast[0] = (u64)(long long)chosen;
      sh.bcast[1] = a;
    }
    __syncthreads();
    const long long chosen = (long long)sh.bcast[0];
    if (chosen < 0) return floor_key;      // everything (above the floor) is below the target
    acc = sh.bcast[1];
    prefix |= ((u64)chosen) << shift;
    __syncthreads();
  }
  return prefix > floor_key ? prefix : floor_key;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(
    int* __restrict__ out, float* __restrict__ logits, int V, long long ld,
    const float* __restrict__ temperature, const int* __restrict__ top_k, const float* __restrict__ top_p,
    const float* __restrict__ min_p, const float* __restrict__ uniform,
    const int* __restrict__ recent, int recent_n, const float* __restrict__ rep_pen,
    const float* __restrict__ freq_pen, const float* __restrict__ pres_pen) {
  __shared__ SampleShared sh;
  const int r = blockIdx.x;
  float* row = logits + (size_t)r * ld;

  // 1. penalties: each distinct recent token once, with its count (sampler.cpp:13-34)
  if (recent && recent_n > 0) {
    const float rp = rep_pen[r], fp = freq_pen[r], pp = pres_pen[r];
    if (rp != 1.0f || fp != 0.0f || pp != 0.0f) {
      const int* rc = recent + (size_t)r * recent_n;
      for (int i = threadIdx.x; i < recent_n; i += blockDim.x) {
        const int tok = rc[i];
        if (tok < 0 || tok >= V) continue;
        int count = 0;
        bool first = true;
        for (int j = 0; j < recent_n; ++j) {
          if (rc[j] == tok) { ++count; if (j < i) first = false; }
        }
        if (!first) continue;
        float l = row[tok];
        if (rp != 1.0f) l = l > 0.f ? l / rp : l * rp;
        l -= (float)count * fp;
        l -= pp;
        row[tok] = l;
      }
      __syncthreads();
    }
  }

  // 2. maximum (and its first index: the greedy answer)
  const float temp = temperature[r];
  float best = -INFINITY;
  int besti = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (v == best && i < besti)) { best = v; besti = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
  }
  __shared__ int si[32];
  if ((threadIdx.x & 31) == 0) { sh.fred[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = besti; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w)
      if (sh.fred[w] > best || (sh.fred[w] == best && si[w] < besti)) { best = sh.fred[w]; besti = si[w]; }
    sh.fred[32] = best;
    si[0] = besti;
  }
  __syncthreads();
  best = sh.fred[32];
  besti = si[0];
  if (temp <= 0.f) {
    if (threadIdx.x == 0) out[r] = besti;
    return;
  }

  // 3. temperature; weights w_i = 2^40 * exp(x_i - x_max), x = logit / temperature
  const float inv_t = 1.0f / temp;
  const float xmax = best * inv_t;
  u64 z = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) z += fixed_weight(row[i] * inv_t, xmax);
  z = block_sum_u64(z, sh);

  // 4. top-k: keep the k largest keys
  u64 floor_key = 0;
  const int k = top_k[r];
  if (k > 0 && k < V) floor_key = radix_threshold(row, V, inv_t, xmax, 0, (u64)k, 0, sh);
  // 5. top-p: the shortest prefix whose mass reaches p * Z
  const float p = top_p[r];
  if (p < 1.0f) {
    u64 target = (u64)((double)p * (double)z);
    if (target < 1) target = 1;
    floor_key = radix_threshold(row, V, inv_t, xmax, floor_key, target, 1, sh);
  }
  // 6. min-p: drop weights below min_p * w_max (w_max = 2^40)
  const float mp = min_p[r];
  const u64 w_floor = mp > 0.f ? (u64)((double)mp * 1099511627776.0) : 0;

  // 7. total weight of the survivors, then the draw in id order
  u64 total = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float x = row[i] * inv_t;
    const u64 w = fixed_weight(x, xmax);
    if (unique_key(x, i) >= floor_key && w >= w_floor) total += w;
  }
  total = block_sum_u64(total, sh);
  if (total == 0) {                       // nothing survived: the reference falls back to argmax
    if (threadIdx.x == 0) out[r] = besti;
    return;
  }
  double u = (double)uniform[r];
  if (u < 0.0) u = 0.0;
  if (u > 0.99999994) u = 0.99999994;
  const u64 target = (u64)(u * (double)total);        // in [0, total)
  u64 running = 0;                                   // weight of all ids before this chunk
  int chosen = -1;
  for (int base = 0; base < V; base += blockDim.x) {
    const int i = base + threadIdx.x;
    u64 w = 0;
    if (i < V) {
      const float x = row[i] * inv_t;
      const u64 ww = fixed_weight(x, xmax);
      if (unique_key(x, i) >= floor_key && ww >= w_floor) w = ww;
    }
    // inclusive scan within the warp, then across warps
    u64 incl = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const u64 t = __shfl_up_sync(0xffffffffu, incl, o);
      if ((threadIdx.x & 31) >= o) incl += t;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 31) sh.red[threadIdx.x >> 5] = incl;
    __syncthreads();
    u64 before = running;
    for (int wv = 0; wv < (threadIdx.x >> 5); ++wv) before += sh.red[wv];
    u64 chunk = 0;
    for (int wv = 0; wv < (blockDim.x >> 5); ++wv) chunk += sh.red[wv];
    const u64 upto = before + incl;
    if (w > 0 && upto > target && upto - w <= target) chosen = i;   // exactly one thread overall
    running += chunk;
    if (running > target) break;          // uniform across the block
  }
  __syncthreads();
  if (chosen >= 0) out[r] = chosen;
}

extern "C" int qv_sample(int* out, float* logits, int rows, int V, long long ld, const float* temperature,
                         const int* top_k, const float* top_p, const float* min_p, const float* uniform,
                         const int* recent, int recent_n, const float* rep_pen, const float* freq_pen,
                         const float* pres_pen, void* stream) {
  if (rows <= 0) return 0;
  sample_kernel<<<rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(
      out, logits, V, ld, temperature, top_k, top_p, min_p, uniform, recent, recent_n, rep_pen, freq_pen,
      pres_pen);
  return qv_launch_status();
}
