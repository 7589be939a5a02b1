// Preparation of queries, keys and values for attention with a norm on every head of q and k, biases on the
// projections and head sizes of q/k and v that may differ: from the fp32 projection row
//   [ q: heads x dim | k: kv_heads x dim | v: kv_heads x vdim | ... ]            (what follows v is not touched)
// of a token to the packed row [q' | k' | v'] with every head padded with zeros to the cache's head size D
// (>= dim and >= vdim), which is the layout the attention kernels read, plus the cache write of k' and v'.
// Padding changes nothing: a zero in q and k adds nothing to a score, and a zero column of v gives a zero
// column of the result, which `gate_mul` drops again.  All arithmetic fp32, one rounding at the end.
//
//   bias     (optional) fp32 [heads*dim + kv_heads*dim + kv_heads*vdim], added to the projection
//   wq, wk   (optional) fp32 [dim]: every head of q (of k) is divided by its root mean square, eps inside the
//            root, and multiplied by this weight, the same for all heads; before the rotation
//   rotation of the first `rotary_dim` numbers of every head of q and k by position * inv_freq[i]; pairing
//            "half": number i with number i + rotary_dim / 2; "interleaved": number 2i with number 2i + 1
//
// gate_mul: out[t, h*vdim + c] = attn[t, h*D + c] * sigmoid(gate[t, h*vdim + c])  (gate fp32, optional: without
//            it the kernel only drops the padding), the input of the output projection.
#include "common.cuh"

using namespace iert;

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;

template <typename T>
__global__ void __launch_bounds__(THREADS)
qkv_prep_kernel(const float* __restrict__ proj, long long ld, const float* __restrict__ bias, T* __restrict__ qkv,
                IertBatchView b, IertKvView c, int heads, int dim, int vdim, const float* __restrict__ inv_freq,
                int rotary_dim, int pairing, const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                int write_cache, int* __restrict__ err) {
  extern __shared__ float sm[];
  pdl_launch_dependents();
  const int D = c.head_dim, nkv = c.kv_heads, half = rotary_dim / 2;
  const int n_heads = heads + 2 * nkv;                 // q heads, k heads, v heads
  float* cs = sm;                                      // [half] cos, [half] sin
  const int width = dim > vdim ? dim : vdim;
  float* rows = sm + rotary_dim;                       // [WARPS][width]
  const int t = blockIdx.x;
  const int s = sequence_of_token(b, t);
  const int slot = s < 0 ? -1 : b.slot_ids[s];
  T* out = qkv + (size_t)t * n_heads * D;
  if (slot < 0) {
    // a padding token: a defined row (the prompt attention kernels read whole tiles of keys and values)
    pdl_wait();
    if (blockIdx.y == 0)
      for (int i = threadIdx.x; i < n_heads * D; i += THREADS) out[i] = from_f32<T>(0.f);
    return;
  }
  const int q_begin = b.cu_q[s], q_len = b.cu_q[s + 1] - q_begin;
  const int pos = b.pos0[s] + (t - q_begin);
  const int final_len = b.pos0[s] + q_len;
  for (int k = threadIdx.x; k < half; k += THREADS) {
    float sn, co;
    sincosf((float)pos * inv_freq[k], &sn, &co);
    cs[k] = co;
    cs[half + k] = sn;
  }
  pdl_wait();
  __syncthreads();
  const bool store = write_cache && pos >= final_len - c.ring_pages * c.page_tokens;
  const float* pr = proj + (size_t)t * ld;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* v = rows + (size_t)warp * width;
  const int qd = heads * dim, kd = nkv * dim;
  for (int h = blockIdx.y * WARPS + warp; h < n_heads; h += gridDim.y * WARPS) {
    const bool is_v = h >= heads + nkv, is_k = !is_v && h >= heads;
    const int n = is_v ? vdim : dim;
    const int src = is_v ? qd + kd + (h - heads - nkv) * vdim : h * dim;       // q and k heads lie one after the other
    float ss = 0.f;
    for (int d = lane; d < n; d += 32) {
      const float x = pr[src + d] + (bias ? bias[src + d] : 0.f);
      v[d] = x;
      ss = fmaf(x, x, ss);
    }
    const float* w = is_v ? nullptr : (is_k ? wk : wq);
    if (w) {
      ss = warp_sum(ss);
      const float r = 1.0f / sqrtf(ss / (float)dim + eps);
      for (int d = lane; d < n; d += 32) v[d] = v[d] * r * w[d];
    }
    __syncwarp();
    if (!is_v) {
      for (int k = lane; k < half; k += 32) {
        const int i0 = pairing == IERT_PAIR_INTERLEAVED ? 2 * k : k;
        const int i1 = pairing == IERT_PAIR_INTERLEAVED ? 2 * k + 1 : k + half;
        const float a = v[i0], bb = v[i1];
        v[i0] = a * cs[k] - bb * cs[half + k];
        v[i1] = bb * cs[k] + a * cs[half + k];
      }
      __syncwarp();
    }
    T* dst = out + (size_t)h * D;
    long long off = -1;
    if (store && (is_k || is_v)) off = kv_row_offset(c, slot, pos, is_k ? h - heads : h - heads - nkv, err);
    T* cache = is_k ? (T*)c.k : (T*)c.v;
    for (int d = lane; d < D; d += 32) {
      const T o = from_f32<T>(d < n ? v[d] : 0.f);
      dst[d] = o;
      if (off >= 0) cache[off + d] = o;
    }
    __syncwarp();
  }
}

__device__ __forceinline__ void store4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float4& v) {
  uint2 w;
  *reinterpret_cast<__nv_bfloat162*>(&w.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&w.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = w;
}

// The same for sizes in whole groups of four (dim, vdim, D, the row stride; 16-byte aligned pointers) and the
// interleaved pairing (or no rotation): a lane holds groups of four consecutive numbers of a head in registers, a pair
// (2i, 2i+1) lies inside one group, so nothing passes through shared memory but the angles; 16-byte loads, 8- or
// 16-byte stores.  CH groups per lane: heads of up to CH * 128 numbers.
template <typename T, int CH>
__global__ void __launch_bounds__(THREADS)
qkv_prep_vec_kernel(const float* __restrict__ proj, long long ld, const float* __restrict__ bias, T* __restrict__ qkv,
                    IertBatchView b, IertKvView c, int heads, int dim, int vdim, const float* __restrict__ inv_freq,
                    int rotary_dim, const float* __restrict__ wq, const float* __restrict__ wk, float eps, int write_cache,
                    int* __restrict__ err) {
  extern __shared__ float sm[];
  pdl_launch_dependents();
  const int D = c.head_dim, nkv = c.kv_heads, half = rotary_dim / 2;
  const int n_heads = heads + 2 * nkv;
  float* cs = sm;                                      // [half] cos, [half] sin
  const int t = blockIdx.x;
  const int s = sequence_of_token(b, t);
  const int slot = s < 0 ? -1 : b.slot_ids[s];
  T* out = qkv + (size_t)t * n_heads * D;
  if (slot < 0) {
    pdl_wait();
    if (blockIdx.y == 0)
      for (int i = threadIdx.x * 4; i < n_heads * D; i += THREADS * 4) store4(out + i, make_float4(0.f, 0.f, 0.f, 0.f));
    return;
  }
  const int q_begin = b.cu_q[s], q_len = b.cu_q[s + 1] - q_begin;
  const int pos = b.pos0[s] + (t - q_begin);
  const int final_len = b.pos0[s] + q_len;
  for (int k = threadIdx.x; k < half; k += THREADS) {
    float sn, co;
    sincosf((float)pos * inv_freq[k], &sn, &co);
    cs[k] = co;
    cs[half + k] = sn;
  }
  pdl_wait();
  __syncthreads();
  const bool store = write_cache && pos >= final_len - c.ring_pages * c.page_tokens;
  const float* pr = proj + (size_t)t * ld;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qd = heads * dim, kd = nkv * dim;
  for (int h = blockIdx.y * WARPS + warp; h < n_heads; h += gridDim.y * WARPS) {
    const bool is_v = h >= heads + nkv, is_k = !is_v && h >= heads;
    const int n = is_v ? vdim : dim;
    const int src = is_v ? qd + kd + (h - heads - nkv) * vdim : h * dim;
    float4 x[CH];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const int e = 4 * (lane + 32 * j);
      x[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (e < n) {
        x[j] = *reinterpret_cast<const float4*>(pr + src + e);
        if (bias) {
          const float4 bb = *reinterpret_cast<const float4*>(bias + src + e);
          x[j].x += bb.x; x[j].y += bb.y; x[j].z += bb.z; x[j].w += bb.w;
        }
        ss += x[j].x * x[j].x + x[j].y * x[j].y + x[j].z * x[j].z + x[j].w * x[j].w;
      }
    }
    const float* w = is_v ? nullptr : (is_k ? wk : wq);
    if (w) {
      ss = warp_sum(ss);
      const float r = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int e = 4 * (lane + 32 * j);
        if (e < n) {
          const float4 ww = *reinterpret_cast<const float4*>(w + e);
          x[j].x = x[j].x * r * ww.x; x[j].y = x[j].y * r * ww.y; x[j].z = x[j].z * r * ww.z; x[j].w = x[j].w * r * ww.w;
        }
      }
    }
    if (!is_v) {
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int k0 = 2 * (lane + 32 * j);                 // the group's pairs: k0 and k0 + 1
        if (k0 < half) {
          const float co = cs[k0], sn = cs[half + k0], a = x[j].x, bb = x[j].y;
          x[j].x = a * co - bb * sn;
          x[j].y = bb * co + a * sn;
        }
        if (k0 + 1 < half) {
          const float co = cs[k0 + 1], sn = cs[half + k0 + 1], a = x[j].z, bb = x[j].w;
          x[j].z = a * co - bb * sn;
          x[j].w = bb * co + a * sn;
        }
      }
    }
    T* dst = out + (size_t)h * D;
    long long off = -1;
    if (store && (is_k || is_v)) off = kv_row_offset(c, slot, pos, is_k ? h - heads : h - heads - nkv, err);
    T* cache = is_k ? (T*)c.k : (T*)c.v;
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const int e = 4 * (lane + 32 * j);
      if (e < D) {                                          // beyond n: the zeros the group was set to
        store4(dst + e, x[j]);
        if (off >= 0) store4(cache + off + e, x[j]);
      }
    }
  }
}

template <typename T>
__global__ void gate_mul_kernel(const T* __restrict__ attn, const float* __restrict__ gate, long long ldg, T* __restrict__ out,
                                int heads, int D, int vdim, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = heads * vdim;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / row;
    const int i = (int)(idx - t * row), h = i / vdim, cidx = i - h * vdim;
    float a = to_f32(attn[(t * heads + h) * D + cidx]);
    if (gate) {
      const float z = gate[t * ldg + i];
      const float e = expf(-fabsf(z));
      a *= z >= 0.f ? 1.0f / (1.0f + e) : e / (1.0f + e);
    }
    out[idx] = from_f32<T>(a);
  }
}

// bf16, eight at a time: vdim and D multiples of 8
__global__ void gate_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ attn, const float* __restrict__ gate, long long ldg,
                                       __nv_bfloat16* __restrict__ out, int heads, int D, int vdim, size_t total8) {
  pdl_launch_dependents();
  pdl_wait();
  const int row8 = heads * vdim / 8;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / row8;
    const int i = (int)(idx - t * row8) * 8, h = i / vdim, cidx = i - h * vdim;
    uint4 a4 = *reinterpret_cast<const uint4*>(attn + (t * heads + h) * D + cidx);
    __nv_bfloat162* ap = reinterpret_cast<__nv_bfloat162*>(&a4);
    if (gate) {
      const float4 g0 = *reinterpret_cast<const float4*>(gate + t * ldg + i);
      const float4 g1 = *reinterpret_cast<const float4*>(gate + t * ldg + i + 4);
      const float z[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = __bfloat1622float2(ap[e]);
        ap[e] = __floats2bfloat162_rn(__fdividef(a.x, 1.0f + __expf(-z[2 * e])), __fdividef(a.y, 1.0f + __expf(-z[2 * e + 1])));
      }
    }
    *reinterpret_cast<uint4*>(out + t * (size_t)heads * vdim + i) = a4;
  }
}

}  // namespace

// proj: fp32 rows (stride ld) that begin with [q | k | v]; qkv: [T, (heads + 2 kv_heads) * D] of `dtype` (= the cache's),
// D = cache->head_dim.
IERT_API int iert_qkv_prep(const float* proj, long long ld, const float* bias, void* qkv, int dtype, const IertBatchView* batch,
                           const IertKvView* cache, int heads, int dim, int vdim, const float* inv_freq, int rotary_dim,
                           int pairing, const float* wq, const float* wk, float eps, int write_cache, int* err,
                           cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  const int D = cache->head_dim;
  if (dim <= 0 || vdim <= 0 || dim > D || vdim > D || rotary_dim < 0 || rotary_dim > dim || (rotary_dim & 1) ||
      cache->dtype != dtype || (pairing != IERT_PAIR_HALF && pairing != IERT_PAIR_INTERLEAVED) || (!wq) != (!wk) ||
      (rotary_dim > 0 && !inv_freq))
    return IERT_BAD_ARGUMENT;
  const size_t smem = ((size_t)rotary_dim + (size_t)WARPS * (dim > vdim ? dim : vdim)) * sizeof(float);
  if (smem > 48 * 1024) return IERT_BAD_ARGUMENT;
  const int n_heads = heads + 2 * cache->kv_heads;
  // many tokens: a block per token; few: the heads of a token over several blocks, a warp's worth each
  const int groups = batch->n_tokens >= 256 ? 1 : (n_heads + WARPS - 1) / WARPS;
  const dim3 grid(batch->n_tokens, groups);
  const int elt = dtype == IERT_F32 ? 4 : 2;
  const bool vec = (pairing == IERT_PAIR_INTERLEAVED || rotary_dim == 0) && dim % 4 == 0 && vdim % 4 == 0 && D % 4 == 0 && D <= 256 &&
                   ld % 4 == 0 && ((uintptr_t)proj & 15) == 0 && (!bias || ((uintptr_t)bias & 15) == 0) &&
                   (!wq || (((uintptr_t)wq & 15) == 0 && ((uintptr_t)wk & 15) == 0)) && ((uintptr_t)qkv % (4 * elt)) == 0 &&
                   ((uintptr_t)cache->k % (4 * elt)) == 0 && ((uintptr_t)cache->v % (4 * elt)) == 0 && (dtype == IERT_F32 || dtype == IERT_BF16);
  if (vec) {
    const size_t vsmem = (size_t)rotary_dim * sizeof(float);
#define GO(T, CH)                                                                                                      \
    launch_dep(qkv_prep_vec_kernel<T, CH>, grid, dim3(THREADS), vsmem, stream, proj, ld, bias, (T*)qkv, *batch, *cache, heads, dim,  \
               vdim, inv_freq, rotary_dim, wq, wk, eps, write_cache, err)
    if (dtype == IERT_F32) { if (D <= 128) GO(float, 1); else GO(float, 2); }
    else { if (D <= 128) GO(__nv_bfloat16, 1); else GO(__nv_bfloat16, 2); }
#undef GO
    return iert_check_launch("qkv_prep");
  }
  if (dtype == IERT_F32)
    launch_dep(qkv_prep_kernel<float>, grid, dim3(THREADS), smem, stream, proj, ld, bias, (float*)qkv, *batch, *cache, heads, dim,
               vdim, inv_freq, rotary_dim, pairing, wq, wk, eps, write_cache, err);
  else if (dtype == IERT_BF16)
    launch_dep(qkv_prep_kernel<__nv_bfloat16>, grid, dim3(THREADS), smem, stream, proj, ld, bias, (__nv_bfloat16*)qkv, *batch,
               *cache, heads, dim, vdim, inv_freq, rotary_dim, pairing, wq, wk, eps, write_cache, err);
  else
    return IERT_BAD_ARGUMENT;
  return iert_check_launch("qkv_prep");
}

// attn: [T, heads * D] of `dtype`; gate: fp32 rows of heads * vdim numbers (stride ldg) or null; out: [T, heads * vdim].
IERT_API int iert_gate_mul(const void* attn, const float* gate, long long ldg, void* out, int dtype, int n_tokens, int heads,
                           int D, int vdim, cudaStream_t stream) {
  if (n_tokens <= 0) return IERT_OK;
  if (heads <= 0 || vdim <= 0 || vdim > D) return IERT_BAD_ARGUMENT;
  const size_t total = (size_t)n_tokens * heads * vdim;
  const int threads = 256;
  const size_t cap = (size_t)iert_sm_count_cached() * 16;
  if (dtype == IERT_BF16 && vdim % 8 == 0 && D % 8 == 0 && ((uintptr_t)attn & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
      (!gate || (((uintptr_t)gate & 15) == 0 && ldg % 4 == 0))) {
    const size_t total8 = total / 8, want = (total8 + threads - 1) / threads;
    launch_dep(gate_mul_bf16x8_kernel, (int)(want < cap ? want : cap), threads, 0, stream, (const __nv_bfloat16*)attn, gate, ldg,
               (__nv_bfloat16*)out, heads, D, vdim, total8);
    return iert_check_launch("gate_mul");
  }
  const size_t want = (total + threads - 1) / threads;
  const int blocks = (int)(want < cap ? want : cap);
  if (dtype == IERT_F32)
    launch_dep(gate_mul_kernel<float>, blocks, threads, 0, stream, (const float*)attn, gate, ldg, (float*)out, heads, D, vdim, total);
  else if (dtype == IERT_BF16)
    launch_dep(gate_mul_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16*)attn, gate, ldg,
               (__nv_bfloat16*)out, heads, D, vdim, total);
  else
    return IERT_BAD_ARGUMENT;
  return iert_check_launch("gate_mul");
}
