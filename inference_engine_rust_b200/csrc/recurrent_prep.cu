// Kernels around the recurrent mixers that do not depend on the state's sizes at compile time.
//
// delta_prep: what the gated delta rule needs per token, from the packed projection of the step:
//   short causal convolution per channel (taps along time, the last column is the current token's,
//   zeros before the sequence's start) + SiLU on the q, k and v channels; q and k made unit vectors
//   per head, x / sqrt(sum x^2 + 1e-6), q also times dim^-1/2; beta = sigmoid(b); the decay
//   g = exp(-exp(A_log) * softplus(a + dt_bias)).  Everything after the projection is fp32.
//   The convolution's history lives in the sequence's state as a ring of `taps` rows: the input of
//   position p is kept in row p % taps, so a step reads rows of earlier positions while it writes
//   its own.  (A step brings either a whole prompt from position 0, which reads no history, or one
//   token, which writes one row and reads the others: no row is read and written in one launch.)
//
// gated_head_norm: each head's read-out divided by its root mean square (eps inside the root),
//   times a weight, times an activation of the gate projection, stored in the run's dtype.
//
// The kernels around the recurrence with a decay per key channel ("wkv"):
//   token_shift   every token's input mixed with the input of the token in front of it, once per reader:
//                 mixed[m][t] = h[t] + (h[t-1] - h[t]) * mu[m]; in front of a sequence's first token stands the row the
//                 state keeps (zeros at the start of a sequence).  fp32 arithmetic, one rounding.
//   wkv_decay     w[t, c] = exp(-exp(w0[c] + sum_l W2[c, l] tanh(z[t, l]))) from the small product z, all fp32;
//                 the same launch leaves each sequence's last input row in the state (the shift has read the old one).
//   wkv_finish    each head's read-out divided by its root mean square (eps inside the root), times a weight, times
//                 silu of the fp32 gate projection, times a fixed factor, stored in the run's dtype.
#include "common.cuh"

using namespace iert;

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

struct DeltaPrepArgs {
  const void* proj;        // [T, ld] run dtype: q [G*D] | k [G*D] | v [H*V] | ...
  long long ld;
  const float* gates;      // [T, gld] fp32: b [H] | a [H]
  long long gld;
  const float* conv_w;     // [C, taps] fp32, C = 2*G*D + H*V
  const float* A_log;      // [H]
  const float* dt_bias;    // [H]
  float* state;            // per slot: conv ring [taps, C] at conv_off
  long long state_stride, conv_off;
  float* qkv;              // out [T, C] fp32
  float* beta;             // out [T, H]
  float* decay;            // out [T, H]
  int G, D, H, V, taps;
};

// One warp per (token, unit), a unit being a q head, a k head or a v head: a lane has a few channels, all its
// loads are independent, and the unit norm is a warp sum: no shared memory, no block barrier, and a step
// of a handful of tokens still spreads over the device.  A block is four tokens of one unit.
constexpr int PREP_MAX_PER_LANE = 16;      // channels of a unit per lane kept in registers (units up to 512 wide)

template <typename T>
__global__ void __launch_bounds__(128) delta_prep_kernel(DeltaPrepArgs a, IertBatchView b) {
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp, unit = blockIdx.y;
  if (t >= b.n_tokens) return;
  const int s = sequence_of_token(b, t);
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  if (slot < 0) return;
  const int GD = a.G * a.D, C = 2 * GD + a.H * a.V, taps = a.taps;
  const bool is_v = unit >= 2 * a.G;
  const int c0 = is_v ? 2 * GD + (unit - 2 * a.G) * a.V : unit * a.D;      // q heads, then k heads, lie back to back
  const int n = is_v ? a.V : a.D;
  const int q_begin = b.cu_q[s], q_end = b.cu_q[s + 1];
  const int pos = b.pos0[s] + (t - q_begin);
  const T* proj = (const T*)a.proj;
  float* ring = a.state + (size_t)slot * a.state_stride + a.conv_off;
  const bool keep = t >= q_end - taps;             // the sequence's newest inputs are its history
  float val[PREP_MAX_PER_LANE];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PREP_MAX_PER_LANE; ++k) {
    const int i = lane + 32 * k;
    val[k] = 0.f;
    if (i < n) {
      const int c = c0 + i;
      float acc = 0.f, now = 0.f;
      for (int j = taps - 1; j >= 0; --j) {        // oldest first
        const int tj = t - j;
        float x = 0.f;
        if (tj >= q_begin) x = to_f32(proj[(size_t)tj * a.ld + c]);
        else if (pos - j >= 0) x = ring[(size_t)((pos - j) % taps) * C + c];
        if (j == 0) now = x;
        acc = fmaf(a.conv_w[(size_t)c * taps + (taps - 1 - j)], x, acc);
      }
      val[k] = silu_f(acc);
      ss = fmaf(val[k], val[k], ss);
      if (keep) ring[(size_t)(pos % taps) * C + c] = now;      // a row no token of this launch reads
    }
  }
  float f = 1.f;
  if (!is_v) {                                      // unit vectors; q also times dim^-1/2
    f = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
    if (unit < a.G) f *= 1.0f / sqrtf((float)a.D);
  }
#pragma unroll
  for (int k = 0; k < PREP_MAX_PER_LANE; ++k) {
    const int i = lane + 32 * k;
    if (i < n) a.qkv[(size_t)t * C + c0 + i] = val[k] * f;
  }
  if (unit == 0)
    for (int h = lane; h < a.H; h += 32) {
      const float gb = a.gates[(size_t)t * a.gld + h], ga = a.gates[(size_t)t * a.gld + a.H + h];
      a.beta[(size_t)t * a.H + h] = sigmoid_f(gb);
      a.decay[(size_t)t * a.H + h] = expf(-expf(a.A_log[h]) * softplus_f(ga + a.dt_bias[h]));
    }
}

// o [T, H*V] fp32; gate: column gate_off + h*V + e of the packed projection; weight index
// h*V + e (per_head = 0) or e (per_head = 1: one vector shared by the heads);
// act 0: SiLU(gate), 1: sigmoid(gate).  One warp per (token, head).
template <typename T>
__global__ void gated_head_norm_kernel(const float* __restrict__ o, const T* __restrict__ proj, long long ld,
                                       int gate_off, const float* __restrict__ w, int per_head, int act,
                                       float eps, T* __restrict__ out, int n_tokens, int H, int V) {
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n_tokens * H) return;
  const int t = warp / H, h = warp - t * H;
  const float* x = o + ((size_t)t * H + h) * V;
  float ss = 0.f;
  for (int e = lane; e < V; e += 32) ss = fmaf(x[e], x[e], ss);
  const float r = 1.0f / sqrtf(warp_sum(ss) / (float)V + eps);
  const T* g = proj + (size_t)t * ld + gate_off + (size_t)h * V;
  T* y = out + ((size_t)t * H + h) * V;
  for (int e = lane; e < V; e += 32) {
    const float gv = to_f32(g[e]);
    const float ga = act == 0 ? silu_f(gv) : sigmoid_f(gv);
    y[e] = from_f32<T>(x[e] * r * w[per_head ? e : h * V + e] * ga);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
token_shift_kernel(const T* __restrict__ h, long long ldh, const float* __restrict__ state, long long state_stride,
                   long long prev_off, const float* __restrict__ mu, int n_mix, int width, T* __restrict__ mixed,
                   IertBatchView b) {
  pdl_wait();
  const int t = blockIdx.x;
  const int s = sequence_of_token(b, t);
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  const size_t plane = (size_t)b.n_tokens * width;
  if (slot < 0) {
    for (int i = threadIdx.x; i < width; i += blockDim.x)
      for (int m = 0; m < n_mix; ++m) mixed[m * plane + (size_t)t * width + i] = from_f32<T>(0.f);
    return;
  }
  const bool first = t == b.cu_q[s];
  const float* kept = state + (size_t)slot * state_stride + prev_off;
  if (sizeof(T) == 2 && width % 8 == 0 && ldh % 8 == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)mixed & 15) == 0 &&
      ((uintptr_t)kept & 15) == 0 && ((uintptr_t)mu & 15) == 0) {
    // eight numbers a thread: 16-byte loads of the row, the row in front and the factors, 16-byte stores per mix
    for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
      float x[8], d[8];
      {
        const uint4 v = *reinterpret_cast<const uint4*>(h + (size_t)t * ldh + i);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(p[e]); x[2 * e] = f.x; x[2 * e + 1] = f.y; }
      }
      if (first) {
        const float4 a = *reinterpret_cast<const float4*>(kept + i), c = *reinterpret_cast<const float4*>(kept + i + 4);
        d[0] = a.x - x[0]; d[1] = a.y - x[1]; d[2] = a.z - x[2]; d[3] = a.w - x[3];
        d[4] = c.x - x[4]; d[5] = c.y - x[5]; d[6] = c.z - x[6]; d[7] = c.w - x[7];
      } else {
        const uint4 v = *reinterpret_cast<const uint4*>(h + (size_t)(t - 1) * ldh + i);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(p[e]); d[2 * e] = f.x - x[2 * e]; d[2 * e + 1] = f.y - x[2 * e + 1]; }
      }
      for (int m = 0; m < n_mix; ++m) {
        const float4 a = *reinterpret_cast<const float4*>(mu + (size_t)m * width + i);
        const float4 c = *reinterpret_cast<const float4*>(mu + (size_t)m * width + i + 4);
        uint4 out;
        __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&out);
        q[0] = __floats2bfloat162_rn(fmaf(d[0], a.x, x[0]), fmaf(d[1], a.y, x[1]));
        q[1] = __floats2bfloat162_rn(fmaf(d[2], a.z, x[2]), fmaf(d[3], a.w, x[3]));
        q[2] = __floats2bfloat162_rn(fmaf(d[4], c.x, x[4]), fmaf(d[5], c.y, x[5]));
        q[3] = __floats2bfloat162_rn(fmaf(d[6], c.z, x[6]), fmaf(d[7], c.w, x[7]));
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(mixed) + m * plane + (size_t)t * width + i) = out;
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float x = to_f32(h[(size_t)t * ldh + i]);
    const float before = first ? kept[i] : to_f32(h[(size_t)(t - 1) * ldh + i]);
    const float d = before - x;
    for (int m = 0; m < n_mix; ++m) mixed[m * plane + (size_t)t * width + i] = from_f32<T>(fmaf(d, mu[(size_t)m * width + i], x));
  }
}

// A block takes DECAY_TOKENS tokens and 256 channels: a thread owns one channel, reads its column of the second matrix
// once (eight loads in flight) and serves all the block's tokens from it, whose tanh rows stand in shared memory.
constexpr int DECAY_TOKENS = 8;

template <typename T>
__global__ void __launch_bounds__(256)
wkv_decay_kernel(const float* __restrict__ z, long long ldz, int L, const float* __restrict__ w2t, const float* __restrict__ w0,
                 int C, float* __restrict__ decay, const T* __restrict__ h, long long ldh, int width,
                 float* __restrict__ state, long long state_stride, long long prev_off, IertBatchView b) {
  extern __shared__ float lora[];          // [DECAY_TOKENS][L]
  __shared__ int keep_slot[DECAY_TOKENS];  // the slot whose kept row token tt becomes (-1: none)
  pdl_wait();
  const int t0 = blockIdx.x * DECAY_TOKENS, n = min(DECAY_TOKENS, b.n_tokens - t0);
  if (threadIdx.x < DECAY_TOKENS) {
    int slot = -1;
    if ((int)threadIdx.x < n) {
      const int t = t0 + threadIdx.x;
      const int s = sequence_of_token(b, t);
      // the sequence's last token of this step is the next step's row in front
      if (s >= 0 && t == b.cu_q[s + 1] - 1) slot = b.slot_ids[s];
    }
    keep_slot[threadIdx.x] = slot;
  }
  for (int i = threadIdx.x; i < DECAY_TOKENS * L; i += blockDim.x) {
    const int tt = i / L, l = i - tt * L;
    lora[tt * L + l] = tt < n ? tanhf(z[(size_t)(t0 + tt) * ldz + l]) : 0.f;
  }
  __syncthreads();
  const int c = blockIdx.y * 256 + threadIdx.x;
  if (c < C) {
    float a[DECAY_TOKENS];
    const float bias = w0[c];
#pragma unroll
    for (int tt = 0; tt < DECAY_TOKENS; ++tt) a[tt] = bias;
    int l = 0;
    if ((L & 3) == 0) {                    // the tokens' rows by 16-byte shared-memory loads, eight weights in flight
      for (; l + 8 <= L; l += 8) {
        float w[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) w[k] = w2t[(size_t)(l + k) * C + c];
#pragma unroll
        for (int tt = 0; tt < DECAY_TOKENS; ++tt) {
          const float4 x0 = *reinterpret_cast<const float4*>(lora + tt * L + l);
          const float4 x1 = *reinterpret_cast<const float4*>(lora + tt * L + l + 4);
          a[tt] = fmaf(w[0], x0.x, a[tt]); a[tt] = fmaf(w[1], x0.y, a[tt]); a[tt] = fmaf(w[2], x0.z, a[tt]); a[tt] = fmaf(w[3], x0.w, a[tt]);
          a[tt] = fmaf(w[4], x1.x, a[tt]); a[tt] = fmaf(w[5], x1.y, a[tt]); a[tt] = fmaf(w[6], x1.z, a[tt]); a[tt] = fmaf(w[7], x1.w, a[tt]);
        }
      }
    }
    for (; l < L; ++l) {
      const float w = w2t[(size_t)l * C + c];
#pragma unroll
      for (int tt = 0; tt < DECAY_TOKENS; ++tt) a[tt] = fmaf(w, lora[tt * L + l], a[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < DECAY_TOKENS; ++tt)
      if (tt < n) decay[(size_t)(t0 + tt) * C + c] = expf(-expf(a[tt]));
  }
  // the kept rows: every block of the token group takes a slice of the width; all loads before the first store
  const int per = (width + gridDim.y - 1) / gridDim.y;
  const int i1 = min(width, ((int)blockIdx.y + 1) * per);
  for (int i = blockIdx.y * per + threadIdx.x; i < i1; i += blockDim.x) {
    float v[DECAY_TOKENS];
#pragma unroll
    for (int tt = 0; tt < DECAY_TOKENS; ++tt)
      if (keep_slot[tt] >= 0) v[tt] = to_f32(h[(size_t)(t0 + tt) * ldh + i]);
#pragma unroll
    for (int tt = 0; tt < DECAY_TOKENS; ++tt)
      if (keep_slot[tt] >= 0) state[(size_t)keep_slot[tt] * state_stride + prev_off + i] = v[tt];
  }
}

template <typename T>
__global__ void wkv_finish_kernel(const float* __restrict__ o, const float* __restrict__ gate, long long ldg,
                                  const float* __restrict__ w, float eps, float out_scale, T* __restrict__ out,
                                  int n_tokens, int H, int V, IertBatchView b) {
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n_tokens * H) return;
  const int t = warp / H, h = warp - t * H;
  T* y = out + ((size_t)t * H + h) * V;
  const float* x = o + ((size_t)t * H + h) * V;
  const float* g = gate + (size_t)t * ldg + (size_t)h * V;
  const bool wide = sizeof(T) == 2 && V % 2 == 0 && V <= 512 && (ldg & 1) == 0 && ((uintptr_t)o & 7) == 0 &&
                    ((uintptr_t)gate & 7) == 0 && ((uintptr_t)w & 7) == 0 && ((uintptr_t)out & 3) == 0;
  // two numbers a lane and load, all asked for before anything waits (also before the look-up of the token's sequence
  // below: a padding token's rows hold leftovers, which are read and dropped)
  float2 xv[8], gv[8], wv[8];
  if (wide) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int e = 2 * lane + 64 * k;
      if (e < V) {
        xv[k] = *reinterpret_cast<const float2*>(x + e);
        gv[k] = *reinterpret_cast<const float2*>(g + e);
        wv[k] = *reinterpret_cast<const float2*>(w + h * V + e);
      }
    }
  }
  const int s = sequence_of_token(b, t);
  if (s < 0 || b.slot_ids[s] < 0) {        // padding: nobody wrote its read-out
    for (int e = lane; e < V; e += 32) y[e] = from_f32<T>(0.f);
    return;
  }
  if (wide) {
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (2 * lane + 64 * k < V) ss = fmaf(xv[k].x, xv[k].x, fmaf(xv[k].y, xv[k].y, ss));
    const float r = out_scale / sqrtf(warp_sum(ss) / (float)V + eps);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int e = 2 * lane + 64 * k;
      if (e < V)
        *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(y) + e) =
            __floats2bfloat162_rn(xv[k].x * r * wv[k].x * silu_f(gv[k].x), xv[k].y * r * wv[k].y * silu_f(gv[k].y));
    }
    return;
  }
  float ss = 0.f;
  for (int e = lane; e < V; e += 32) ss = fmaf(x[e], x[e], ss);
  const float r = out_scale / sqrtf(warp_sum(ss) / (float)V + eps);
  for (int e = lane; e < V; e += 32) y[e] = from_f32<T>(x[e] * r * w[h * V + e] * silu_f(g[e]));
}

}  // namespace

// h: [T, ldh] the step's input rows (run dtype); state: fp32 per slot, the kept row at prev_off; mu: fp32 [n_mix, width];
// mixed: [n_mix, T, width] run dtype.
IERT_API int iert_token_shift(const void* h, int dtype, long long ldh, const float* state, long long state_stride,
                              long long prev_off, const float* mu, int n_mix, int width, void* mixed,
                              const IertBatchView* batch, cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  if (n_mix <= 0 || width <= 0) return IERT_BAD_ARGUMENT;
  if (dtype == IERT_F32)
    launch_dep(token_shift_kernel<float>, dim3(batch->n_tokens), dim3(256), 0, stream, (const float*)h, ldh, state, state_stride,
               prev_off, mu, n_mix, width, (float*)mixed, *batch);
  else if (dtype == IERT_BF16)
    launch_dep(token_shift_kernel<__nv_bfloat16>, dim3(batch->n_tokens), dim3(256), 0, stream, (const __nv_bfloat16*)h, ldh, state,
               state_stride, prev_off, mu, n_mix, width, (__nv_bfloat16*)mixed, *batch);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("token_shift");
}

// z: fp32 [T, ldz] (L used); w2t: fp32 [L, C] (the second matrix, transposed); w0: fp32 [C]; decay: fp32 [T, C].
// h / state as for iert_token_shift: the last row of every sequence is stored at prev_off.
IERT_API int iert_wkv_decay(const float* z, long long ldz, int L, const float* w2t, const float* w0, int C, float* decay,
                            const void* h, int dtype, long long ldh, int width, float* state, long long state_stride,
                            long long prev_off, const IertBatchView* batch, cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  if (L <= 0 || L > 1024 || C <= 0 || width <= 0) return IERT_BAD_ARGUMENT;
  const size_t smem = (size_t)DECAY_TOKENS * L * sizeof(float);
  const dim3 grid((batch->n_tokens + DECAY_TOKENS - 1) / DECAY_TOKENS, (C + 255) / 256);
  if (dtype == IERT_F32)
    launch_dep(wkv_decay_kernel<float>, grid, dim3(256), smem, stream, z, ldz, L, w2t, w0, C, decay,
               (const float*)h, ldh, width, state, state_stride, prev_off, *batch);
  else if (dtype == IERT_BF16)
    launch_dep(wkv_decay_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, z, ldz, L, w2t, w0, C, decay,
               (const __nv_bfloat16*)h, ldh, width, state, state_stride, prev_off, *batch);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("wkv_decay");
}

// o: fp32 [T, H*V]; gate: fp32 [T, ldg] (H*V used); w: fp32 [H*V]; out: [T, H*V] in `dtype`.
IERT_API int iert_wkv_finish(const float* o, const float* gate, long long ldg, const float* w, float eps, float out_scale,
                             void* out, int dtype, const IertBatchView* batch, int H, int V, cudaStream_t stream) {
  const int n_tokens = batch->n_tokens;
  if (n_tokens <= 0) return IERT_OK;
  if (H <= 0 || V <= 0) return IERT_BAD_ARGUMENT;
  const unsigned blocks = (unsigned)(((long long)n_tokens * H + 3) / 4);
  if (dtype == IERT_F32)
    launch_dep(wkv_finish_kernel<float>, dim3(blocks), dim3(128), 0, stream, o, gate, ldg, w, eps, out_scale, (float*)out, n_tokens, H, V, *batch);
  else if (dtype == IERT_BF16)
    launch_dep(wkv_finish_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, o, gate, ldg, w, eps, out_scale,
               (__nv_bfloat16*)out, n_tokens, H, V, *batch);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("wkv_finish");
}

IERT_API int iert_delta_prep(const void* proj, int dtype, long long ld, const float* gates, long long gld,
                             const float* conv_w, const float* A_log, const float* dt_bias, float* state,
                             long long state_stride, long long conv_off, float* qkv, float* beta, float* decay,
                             int G, int D, int H, int V, int taps, const IertBatchView* batch, cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  const long long C = 2LL * G * D + (long long)H * V;
  if (G <= 0 || D <= 0 || H <= 0 || V <= 0 || taps <= 0 || D > 32 * PREP_MAX_PER_LANE || V > 32 * PREP_MAX_PER_LANE ||
      2 * G + H > 65535)
    return IERT_BAD_ARGUMENT;
  DeltaPrepArgs a = {proj, ld, gates, gld, conv_w, A_log, dt_bias, state, state_stride, conv_off, qkv, beta, decay,
                     G, D, H, V, taps};
  (void)C;
  const size_t smem = 0;
  const dim3 grid((batch->n_tokens + 3) / 4, 2 * G + H);
  if (dtype == IERT_F32) launch_dep(delta_prep_kernel<float>, grid, dim3(128), smem, stream, a, *batch);
  else if (dtype == IERT_BF16) launch_dep(delta_prep_kernel<__nv_bfloat16>, grid, dim3(128), smem, stream, a, *batch);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("delta_prep");
}

IERT_API int iert_gated_head_norm(const float* o, const void* proj, int dtype, long long ld, int gate_off,
                                  const float* w, int per_head, int act, float eps, void* out, int n_tokens,
                                  int H, int V, cudaStream_t stream) {
  if (n_tokens <= 0) return IERT_OK;
  if (H <= 0 || V <= 0) return IERT_BAD_ARGUMENT;
  const long long warps = (long long)n_tokens * H;
  const unsigned blocks = (unsigned)((warps + 3) / 4);
  if (dtype == IERT_F32)
    launch_dep(gated_head_norm_kernel<float>, dim3(blocks), dim3(128), 0, stream, o, (const float*)proj, ld, gate_off, w,
               per_head, act, eps, (float*)out, n_tokens, H, V);
  else if (dtype == IERT_BF16)
    launch_dep(gated_head_norm_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, o, (const __nv_bfloat16*)proj,
               ld, gate_off, w, per_head, act, eps, (__nv_bfloat16*)out, n_tokens, H, V);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("gated_head_norm");
}
