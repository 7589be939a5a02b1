// Attention whose keys and values are expanded from one low-rank row c per token (the only thing
// the cache keeps), without positions, with a sink in the softmax's denominator:
//
//   weights  p_j = exp(s_j - M) / (sum_j exp(s_j - M) + exp(sink_h - M)),  s_j = (q . k_j) * scale,
//   M = max(max_j s_j, sink_h); the sink is a bare logit per head: it enters the denominator unscaled and
//   adds nothing to the numerator.
//
// latent_norm_store: RMS norm (plain weight, eps inside the root) of the two down-projections of a
//   token (query latent, key/value latent), fp32 statistics; the key/value latent is also written to
//   the paged cache (kv_heads = 1, head_dim = rank).
// latent_attention_prompt: a prompt that starts at position 0 attends over the step's own expanded
//   keys and values, packed per token as q [H*D] | k [H*D] | v [H*V] (D and V may differ).
// latent_attention_decode: one token per sequence over the cached latents, in the absorbed form:
//   qa = W_uk[h]^T q  (rank numbers), s_j = (qa . c_j) * scale, l = sum_j p_j c_j, o = W_uv[h] l.
//   Nothing is expanded per cached position.  With a rotated part of R numbers a cached row is [c_j | r_j] (r_j: one
//   rotated key part shared by all heads), a query head is [unrotated D | rotated R], and s_j = (qa . c_j + q_rot . r_j)
//   * scale; the weighted sum still runs over the latents alone.  `gate` (fp32 [T, H], optional) multiplies head h's result.
// latent_prep / head_gate_mul: the preparation of that variant's rows and the gate on a prompt's result (below).
// All arithmetic is fp32; one block per (token, head); keys are visited in chunks with a running
// maximum and sum, so the memory needed does not grow with the context.
#include "common.cuh"

using namespace iert;

namespace {

constexpr int THREADS = 128;
constexpr int MAX_PER_THREAD = 8;       // value size / rank up to 1024

template <typename T>
__global__ void latent_norm_store_kernel(const float* __restrict__ x, long long ldx, int q_rank, int kv_rank,
                                         const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                                         T* __restrict__ cq, T* __restrict__ c, IertBatchView b, IertKvView kv,
                                         int store, int* __restrict__ err) {
  __shared__ float scratch[33];
  pdl_wait();
  const int t = blockIdx.x;
  const int s = sequence_of_token(b, t);
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  if (slot < 0) return;
  const float* row = x + (size_t)t * ldx;
  float ss = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
  const float rq = 1.0f / sqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cq[(size_t)t * q_rank + i] = from_f32<T>(row[i] * rq * wq[i]);
  ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) ss = fmaf(row[q_rank + i], row[q_rank + i], ss);
  const float rk = 1.0f / sqrtf(block_sum(ss, scratch) / (float)kv_rank + eps);
  T* dst = nullptr;
  if (store) {
    const int pos = b.pos0[s] + (t - b.cu_q[s]);
    const long long off = kv_row_offset(kv, slot, pos, 0, err);
    if (off >= 0) dst = (T*)kv.k + off;
  }
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
    const T v = from_f32<T>(row[q_rank + i] * rk * wkv[i]);
    c[(size_t)t * kv_rank + i] = v;
    if (dst) dst[i] = v;
  }
}

// Shared by both attention kernels: one chunk of scores is in sc (this thread's key) -> running
// maximum / sum update; returns the factor for what was accumulated so far and leaves p in p_s.
__device__ __forceinline__ float softmax_chunk(float sc, float& m, float& l, float* p_s, float* scratch) {
  const float m_new = fmaxf(m, block_max(sc, scratch));
  const float p = sc == -INFINITY ? 0.f : expf(sc - m_new);
  const float alpha = m == -INFINITY ? 0.f : expf(m - m_new);
  l = l * alpha + block_sum(p, scratch);
  m = m_new;
  p_s[threadIdx.x] = p;
  __syncthreads();
  return alpha;
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
latent_attention_prompt_kernel(const T* __restrict__ qkv, long long ld, T* __restrict__ out, IertBatchView b,
                               int H, int D, int V, float scale, const float* __restrict__ sink) {
  extern __shared__ float smem[];
  float* q_s = smem;                  // [D]
  float* p_s = smem + D;              // [THREADS]
  float* scratch = p_s + THREADS;     // [33]
  pdl_wait();
  const int t = blockIdx.x, head = blockIdx.y;
  T* o = out + ((size_t)t * H + head) * V;
  const int s = sequence_of_token(b, t);
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  if (slot < 0) {
    for (int e = threadIdx.x; e < V; e += THREADS) o[e] = from_f32<T>(0.f);
    return;
  }
  const int q_begin = b.cu_q[s];
  const int pos = t - q_begin;                       // the prompt starts at position 0
  const T* q = qkv + (size_t)t * ld + (size_t)head * D;
  for (int d = threadIdx.x; d < D; d += THREADS) q_s[d] = to_f32(q[d]);
  __syncthreads();
  const float snk = sink ? sink[head] : -INFINITY;
  float m = snk, l = sink ? 1.f : 0.f;               // the sink: a term exp(sink - M) with no value
  float acc[MAX_PER_THREAD];
#pragma unroll
  for (int i = 0; i < MAX_PER_THREAD; ++i) acc[i] = 0.f;
  for (int j0 = 0; j0 <= pos; j0 += THREADS) {
    const int j = j0 + threadIdx.x;
    float sc = -INFINITY;
    if (j <= pos) {
      const T* k = qkv + (size_t)(q_begin + j) * ld + (size_t)(H + head) * D;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot = fmaf(q_s[d], to_f32(k[d]), dot);
      sc = dot * scale;
    }
    const float alpha = softmax_chunk(sc, m, l, p_s, scratch);
    const int n_in = min(THREADS, pos - j0 + 1);
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
      const int e = threadIdx.x + i * THREADS;
      if (e >= V) break;
      float a = acc[i] * alpha;
      const T* v = qkv + (size_t)(q_begin + j0) * ld + (size_t)2 * H * D + (size_t)head * V + e;
      for (int jj = 0; jj < n_in; ++jj) a = fmaf(p_s[jj], to_f32(v[(size_t)jj * ld]), a);
      acc[i] = a;
    }
    __syncthreads();
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < MAX_PER_THREAD; ++i) {
    const int e = threadIdx.x + i * THREADS;
    if (e < V) o[e] = from_f32<T>(acc[i] * inv);
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
latent_attention_decode_kernel(const T* __restrict__ q, long long ldq, const T* __restrict__ w_uk,
                               const T* __restrict__ w_uv, T* __restrict__ out, IertBatchView b, IertKvView kv,
                               int H, int D, int R, int V, float scale, const float* __restrict__ sink,
                               const float* __restrict__ gate, int* __restrict__ err) {
  extern __shared__ float smem[];
  const int width = kv.head_dim, rank = width - R;   // a cached row: the latent [rank] | the shared rotated key part [R]
  float* qa = smem;                   // [width]: the query in the latent's coordinates | its rotated part
  float* lat = qa + width;            // [rank]: the weighted sum of latents
  float* q_s = lat + rank;            // [D + R]
  float* p_s = q_s + D + R;           // [THREADS]
  float* scratch = p_s + THREADS;     // [33]
  pdl_wait();
  const int t = blockIdx.x, head = blockIdx.y;
  T* o = out + ((size_t)t * H + head) * V;
  const int s = sequence_of_token(b, t);
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  if (slot < 0) {
    for (int e = threadIdx.x; e < V; e += THREADS) o[e] = from_f32<T>(0.f);
    return;
  }
  const int pos = b.pos0[s] + (t - b.cu_q[s]);
  for (int d = threadIdx.x; d < D + R; d += THREADS) q_s[d] = to_f32(q[(size_t)t * ldq + (size_t)head * (D + R) + d]);
  __syncthreads();
  for (int r = threadIdx.x; r < rank; r += THREADS) {
    const T* w = w_uk + (size_t)head * D * rank + r;
    float a = 0.f;
    for (int d = 0; d < D; ++d) a = fmaf(q_s[d], to_f32(w[(size_t)d * rank]), a);
    qa[r] = a;
  }
  for (int i = threadIdx.x; i < R; i += THREADS) qa[rank + i] = q_s[D + i];
  __syncthreads();
  const float snk = sink ? sink[head] : -INFINITY;
  float m = snk, l = sink ? 1.f : 0.f;
  float acc[MAX_PER_THREAD];
#pragma unroll
  for (int i = 0; i < MAX_PER_THREAD; ++i) acc[i] = 0.f;
  const T* cache = (const T*)kv.k;
  for (int j0 = 0; j0 <= pos; j0 += THREADS) {
    const int j = j0 + threadIdx.x;
    float sc = -INFINITY;
    if (j <= pos) {
      const long long off = kv_row_offset(kv, slot, j, 0, err);
      if (off >= 0) {
        const T* c = cache + off;
        float dot = 0.f;
        for (int r = 0; r < width; ++r) dot = fmaf(qa[r], to_f32(c[r]), dot);
        sc = dot * scale;
      }
    }
    const float alpha = softmax_chunk(sc, m, l, p_s, scratch);
    const int n_in = min(THREADS, pos - j0 + 1);
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
      const int r = threadIdx.x + i * THREADS;
      if (r >= rank) break;
      float a = acc[i] * alpha;
      for (int jj = 0; jj < n_in; ++jj) {
        const float pj = p_s[jj];
        if (pj == 0.f) continue;
        const long long off = kv_row_offset(kv, slot, j0 + jj, 0, nullptr);
        if (off < 0) continue;
        a = fmaf(pj, to_f32(cache[off + r]), a);
      }
      acc[i] = a;
    }
    __syncthreads();
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < MAX_PER_THREAD; ++i) {
    const int r = threadIdx.x + i * THREADS;
    if (r < rank) lat[r] = acc[i] * inv;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = warp; e < V; e += THREADS / 32) {
    const T* w = w_uv + ((size_t)head * V + e) * rank;
    float a = 0.f;
    for (int r = lane; r < rank; r += 32) a = fmaf(to_f32(w[r]), lat[r], a);
    a = warp_sum(a);
    if (lane == 0) o[e] = from_f32<T>(gate ? a * gate[(size_t)t * H + head] : a);
  }
}

// The step's rows of latent attention with a rotated part, from one fp32 projection row per token
//   x = [ q: H heads of (D unrotated | R rotated) | down: rank latent numbers | R rotated key numbers | H gate logits ]
// to what the attention kernels read:
//   c_ext [T, rank + R]   RMS-normed latent (plain weight, eps inside the root) | rotated key part; also the cache row
//   q_out [T, H, q_head]  per head (D unrotated | R rotated | zeros up to q_head)
//   gate_out [T, H]       sigmoid(gate logit) * out_scale  (fp32), if the layer has a gate
// Angles are position * inv_freq[i] in fp32 with the precise sine and cosine; pairs are neighbours (2i, 2i+1) or
// halves (i, i + R/2).  One block per token; all arithmetic fp32, one rounding at the store.
template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ x, long long ldx, int H, int D, int R, int rank,
                                   const float* __restrict__ wkv, float eps, const float* __restrict__ inv_freq, int pairing,
                                   int has_gate, float out_scale, T* __restrict__ c_ext, T* __restrict__ q_out, long long ldq,
                                   int q_head, float* __restrict__ gate_out, IertBatchView b, IertKvView kv, int store,
                                   int* __restrict__ err) {
  __shared__ float scratch[33];
  pdl_wait();
  const int t = blockIdx.x;
  const int s = sequence_of_token(b, t);
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  T* qrow = q_out + (size_t)t * ldq;
  if (slot < 0) {                       // padding: rows of zeros, nothing stored
    for (int i = threadIdx.x; i < H * q_head; i += blockDim.x) qrow[i] = from_f32<T>(0.f);
    for (int i = threadIdx.x; i < rank + R; i += blockDim.x) c_ext[(size_t)t * (rank + R) + i] = from_f32<T>(0.f);
    if (has_gate) for (int i = threadIdx.x; i < H; i += blockDim.x) gate_out[(size_t)t * H + i] = 0.f;
    return;
  }
  const int pos = b.pos0[s] + (t - b.cu_q[s]);
  const float* row = x + (size_t)t * ldx;
  const float* down = row + (size_t)H * (D + R);
  const float* glog = down + rank + R;
  const int half = R / 2;
  // the rotated partner and sign of element i of a rotated part: out = v[i] cos - v[partner] sin for the first of a pair
  auto rotated = [&](const float* v, int i) -> float {
    int k, first;
    if (pairing == IERT_PAIR_INTERLEAVED) { k = i >> 1; first = !(i & 1); }
    else { k = i < half ? i : i - half; first = i < half; }
    const int other = pairing == IERT_PAIR_INTERLEAVED ? (i ^ 1) : (first ? i + half : i - half);
    float sn, cs;
    sincosf((float)pos * inv_freq[k], &sn, &cs);
    return first ? v[i] * cs - v[other] * sn : v[i] * cs + v[other] * sn;
  };
  for (int i = threadIdx.x; i < H * q_head; i += blockDim.x) {
    const int h = i / q_head, d = i - h * q_head;
    const float* qh = row + (size_t)h * (D + R);
    float v = 0.f;
    if (d < D) v = qh[d];
    else if (d < D + R) v = rotated(qh + D, d - D);
    qrow[i] = from_f32<T>(v);
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(down[i], down[i], ss);
  const float rk = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
  T* dst = nullptr;
  if (store && pos >= b.pos0[s] + (b.cu_q[s + 1] - b.cu_q[s]) - kv.ring_pages * kv.page_tokens) {
    const long long off = kv_row_offset(kv, slot, pos, 0, err);
    if (off >= 0) dst = (T*)kv.k + off;
  }
  for (int i = threadIdx.x; i < rank + R; i += blockDim.x) {
    const T v = from_f32<T>(i < rank ? down[i] * rk * wkv[i] : rotated(down + rank, i - rank));
    c_ext[(size_t)t * (rank + R) + i] = v;
    if (dst) dst[i] = v;
  }
  if (has_gate)
    for (int i = threadIdx.x; i < H; i += blockDim.x) gate_out[(size_t)t * H + i] = out_scale / (1.0f + expf(-glog[i]));
}

// out[t, h, :V] = attn[t, h, :V] * gate[t, h]: drops the padding of heads of `head` numbers and applies the gate.
template <typename T>
__global__ void head_gate_mul_kernel(const T* __restrict__ attn, int head, T* __restrict__ out, int V, int H,
                                     const float* __restrict__ gate, IertBatchView b) {
  pdl_wait();
  const int t = blockIdx.x;
  const int s = sequence_of_token(b, t);
  if (s < 0 || b.slot_ids[s] < 0) {        // padding: its attention rows may never have been written
    for (int i = threadIdx.x; i < H * V; i += blockDim.x) out[(size_t)t * H * V + i] = from_f32<T>(0.f);
    return;
  }
  if (sizeof(T) == 2 && V % 8 == 0 && head % 8 == 0 && ((uintptr_t)attn & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    for (int i = threadIdx.x * 8; i < H * V; i += blockDim.x * 8) {      // eight numbers of one head at a time
      const int h = i / V, e = i - h * V;
      const float g = gate ? gate[(size_t)t * H + h] : 1.f;
      uint4 v = *reinterpret_cast<const uint4*>(attn + ((size_t)t * H + h) * head + e);
      __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(p2[k]);
        p2[k] = __floats2bfloat162_rn(f.x * g, f.y * g);
      }
      *reinterpret_cast<uint4*>(out + (size_t)t * H * V + i) = v;
    }
    return;
  }
  for (int i = threadIdx.x; i < H * V; i += blockDim.x) {
    const int h = i / V, e = i - h * V;
    const float g = gate ? gate[(size_t)t * H + h] : 1.f;
    out[(size_t)t * H * V + i] = from_f32<T>(to_f32(attn[((size_t)t * H + h) * head + e]) * g);
  }
}

}  // namespace

// x: fp32 [T, ldx] = query latent [q_rank] | key/value latent [kv_rank], before their norms.
IERT_API int iert_latent_norm_store(const float* x, long long ldx, int q_rank, int kv_rank, const float* wq,
                                    const float* wkv, float eps, void* cq, void* c, int dtype,
                                    const IertBatchView* batch, const IertKvView* kv, int store, int* err,
                                    cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  if (q_rank <= 0 || kv_rank <= 0 || (store && (kv->head_dim != kv_rank || kv->kv_heads != 1 || kv->dtype != dtype)))
    return IERT_BAD_ARGUMENT;
  if (dtype == IERT_F32)
    launch_dep(latent_norm_store_kernel<float>, dim3(batch->n_tokens), dim3(128), 0, stream, x, ldx, q_rank, kv_rank, wq,
               wkv, eps, (float*)cq, (float*)c, *batch, *kv, store, err);
  else if (dtype == IERT_BF16)
    launch_dep(latent_norm_store_kernel<__nv_bfloat16>, dim3(batch->n_tokens), dim3(128), 0, stream, x, ldx, q_rank,
               kv_rank, wq, wkv, eps, (__nv_bfloat16*)cq, (__nv_bfloat16*)c, *batch, *kv, store, err);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("latent_norm_store");
}

// qkv: [T, ld] packed q [H*D] | k [H*D] | v [H*V]; out [T, H*V]; sink fp32 [H] or nullptr.
IERT_API int iert_latent_attention_prompt(const void* qkv, long long ld, void* out, int dtype,
                                          const IertBatchView* batch, int H, int D, int V, float scale,
                                          const float* sink, cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  if (H <= 0 || H > 65535 || D <= 0 || V <= 0 || V > THREADS * MAX_PER_THREAD || D > 8192) return IERT_BAD_ARGUMENT;
  dim3 grid(batch->n_tokens, H);
  const size_t smem = (size_t)(D + THREADS + 33) * sizeof(float);
  if (dtype == IERT_F32)
    launch_dep(latent_attention_prompt_kernel<float>, grid, dim3(THREADS), smem, stream, (const float*)qkv, ld,
               (float*)out, *batch, H, D, V, scale, sink);
  else if (dtype == IERT_BF16)
    launch_dep(latent_attention_prompt_kernel<__nv_bfloat16>, grid, dim3(THREADS), smem, stream,
               (const __nv_bfloat16*)qkv, ld, (__nv_bfloat16*)out, *batch, H, D, V, scale, sink);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("latent_attention_prompt");
}

// q: [T, ldq] (H*D per token); w_uk [H*D, rank], w_uv [H*V, rank] row-major in the run's dtype;
// the cache view holds the latents (k only).  out [T, H*V].
IERT_API int iert_latent_attention_decode(const void* q, long long ldq, const void* w_uk, const void* w_uv, void* out,
                                          int dtype, const IertBatchView* batch, const IertKvView* kv, int H, int D,
                                          int R, int V, float scale, const float* sink, const float* gate, int* err,
                                          cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  const int rank = kv->head_dim - R;
  if (H <= 0 || H > 65535 || D <= 0 || R < 0 || V <= 0 || rank <= 0 || rank > THREADS * MAX_PER_THREAD || kv->kv_heads != 1 ||
      kv->dtype != dtype || 2 * rank + D + 2 * R > 10000)
    return IERT_BAD_ARGUMENT;
  dim3 grid(batch->n_tokens, H);
  const size_t smem = (size_t)(2 * rank + D + 2 * R + THREADS + 33) * sizeof(float);
  if (dtype == IERT_F32)
    launch_dep(latent_attention_decode_kernel<float>, grid, dim3(THREADS), smem, stream, (const float*)q, ldq,
               (const float*)w_uk, (const float*)w_uv, (float*)out, *batch, *kv, H, D, R, V, scale, sink, gate, err);
  else if (dtype == IERT_BF16)
    launch_dep(latent_attention_decode_kernel<__nv_bfloat16>, grid, dim3(THREADS), smem, stream,
               (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)w_uk, (const __nv_bfloat16*)w_uv,
               (__nv_bfloat16*)out, *batch, *kv, H, D, R, V, scale, sink, gate, err);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("latent_attention_decode");
}

// x: fp32 [T, ldx] = q [H * (D + R)] | latent [rank] | rotated key part [R] | gate logits [H] (if has_gate).
// c_ext [T, rank + R], q_out [T, H * q_head] with row stride ldq (q_head >= D + R) in `dtype`; gate_out fp32 [T, H]; inv_freq fp32 [R / 2].
// With `store` the rows of c_ext also go to the cache (kv_heads 1, head_dim rank + R, keys only).
IERT_API int iert_latent_prep(const float* x, long long ldx, int H, int D, int R, int rank, const float* wkv, float eps,
                              const float* inv_freq, int pairing, int has_gate, float out_scale, void* c_ext, void* q_out,
                              long long ldq, int q_head, float* gate_out, int dtype, const IertBatchView* batch, const IertKvView* kv,
                              int store, int* err, cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  if (H <= 0 || D < 0 || R < 0 || (R & 1) || rank <= 0 || q_head < D + R || ldq < (long long)H * q_head || (R > 0 && !inv_freq) || (has_gate && !gate_out) ||
      (pairing != IERT_PAIR_HALF && pairing != IERT_PAIR_INTERLEAVED) ||
      (store && (kv->head_dim != rank + R || kv->kv_heads != 1 || kv->dtype != dtype)))
    return IERT_BAD_ARGUMENT;
  if (dtype == IERT_F32)
    launch_dep(latent_prep_kernel<float>, dim3(batch->n_tokens), dim3(256), 0, stream, x, ldx, H, D, R, rank, wkv, eps, inv_freq,
               pairing, has_gate, out_scale, (float*)c_ext, (float*)q_out, ldq, q_head, gate_out, *batch, *kv, store, err);
  else if (dtype == IERT_BF16)
    launch_dep(latent_prep_kernel<__nv_bfloat16>, dim3(batch->n_tokens), dim3(256), 0, stream, x, ldx, H, D, R, rank, wkv, eps,
               inv_freq, pairing, has_gate, out_scale, (__nv_bfloat16*)c_ext, (__nv_bfloat16*)q_out, ldq, q_head, gate_out, *batch,
               *kv, store, err);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("latent_prep");
}

// attn [T, H * head] -> out [T, H * V] (V <= head), times gate [T, H] (fp32, optional).
IERT_API int iert_head_gate_mul(const void* attn, int head, void* out, int V, int H, const float* gate, int dtype,
                                const IertBatchView* batch, cudaStream_t stream) {
  const int n_tokens = batch->n_tokens;
  if (n_tokens <= 0) return IERT_OK;
  if (H <= 0 || V <= 0 || head < V) return IERT_BAD_ARGUMENT;
  if (dtype == IERT_F32)
    launch_dep(head_gate_mul_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, (const float*)attn, head, (float*)out, V, H, gate, *batch);
  else if (dtype == IERT_BF16)
    launch_dep(head_gate_mul_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, stream, (const __nv_bfloat16*)attn, head,
               (__nv_bfloat16*)out, V, H, gate, *batch);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("head_gate_mul");
}
