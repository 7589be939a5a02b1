// Recurrences with a matrix state per head, S [DIM x V] in fp32, carried from token to token in the
// sequence's state.  Compiled per key size (-DDIM=...), like the attention kernels per head size.
//
// Work split: a column j of S never meets another column, so a CTA owns (sequence, head, a run of
// columns) and a thread owns RPT = ceil(DIM / R) rows of one column in registers (rows r, r + R, ...: the
// lanes of a column read neighbouring words of a token's k and q, so shared memory serves them without bank
// conflicts); the R threads of a column are neighbouring lanes and add their partial dot products by shuffles.  R is chosen at the
// launch: the tokens of a sequence are a chain, so all the parallelism there is lies in heads x columns x
// R, and a single prompt wants many lanes per column (more warps per SM to hide the chain's latency)
// where a batch of sequences is served best by few (fewer shuffles and shared-memory reads per FMA).
// A CTA walks its sequence's tokens in order; the tokens' vectors come through shared memory CHUNK
// tokens at a time, fetched (and converted) by two warps that do nothing else into the buffer the
// computing warps are not reading, so that those never wait for memory: one barrier per chunk.
// State is read when the CTA starts and written back when it ends, so a step of one token and a
// prompt of thousands run the same code.
//
//   gated delta rule, per token:   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   mLSTM, per token:  m' = max(f + m, i);  S <- e^(f+m-m') S + e^(i-m') k v^T;  n likewise with k;
//                      o = S^T q / (max(|n . q|, e^(-m')) + 1e-6),  m starts at 0
//       with i = cap tanh((zi + bi) / cap),  f = logsigmoid(cap tanh((zf + bf) / cap))
//   wkv (decay per key channel, a bonus for the current token), per token:
//                      o = (S + diag(u) k v^T)^T r;  S <- diag(w) S + k v^T
#include "common.cuh"

#include <stdlib.h>

using namespace iert;

#ifndef DIM
#error "compile with -DDIM=<rows of the state matrix>"
#endif

namespace {

constexpr int fewest_lanes() {                 // the fewest lanes per column that keep a thread's rows at 32 or fewer
  int r = 1;
  while ((DIM + r - 1) / r > 32 && r < 32) r *= 2;
  return r;
}
constexpr int R_MIN = fewest_lanes();
constexpr int CHUNK = DIM <= 128 ? 8 : DIM <= 256 ? 4 : DIM <= 512 ? 2 : 1;
constexpr int LOADERS = 64;                    // threads of a CTA that only fetch

template <int R>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = R / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct DeltaArgs {
  const float* qkv;      // [T, C] fp32: q [G*DIM] | k [G*DIM] | v [H*V]   (from delta_prep)
  const float* beta;     // [T, H]
  const float* decay;    // [T, H]
  float* state;          // per slot at s_off: S [H, DIM, V]
  long long state_stride, s_off;
  float* o;              // [T, H*V] fp32
  int G, H, V, cols;
};

template <int R>
__global__ void __launch_bounds__(256 + LOADERS) delta_recur_kernel(DeltaArgs a, IertBatchView b) {
  constexpr int RPT = (DIM + R - 1) / R;
  __shared__ __align__(16) float k_s[2][CHUNK][DIM], q_s[2][CHUNK][DIM], v_s[2][CHUNK][256], bg_s[2][CHUNK][2];
  pdl_wait();
  const int s = blockIdx.x, head = blockIdx.y, c0 = blockIdx.z * a.cols;
  const int slot = b.slot_ids[s];
  const int t0 = b.cu_q[s], t1 = b.cu_q[s + 1];
  if (slot < 0 || t1 <= t0) return;
  const int workers = blockDim.x - LOADERS;
  const bool loader = (int)threadIdx.x >= workers;
  const int col = threadIdx.x / R, r = threadIdx.x % R;
  const int j = c0 + col;
  const bool live = !loader && col < a.cols && j < a.V;
  const int g = head / (a.H / a.G);
  const int GD = a.G * DIM, C = 2 * GD + a.H * a.V;
  auto fetch = [&](int buf, int tc, int tid, int nthreads) {
    const int n = min(CHUNK, t1 - tc);
    if (DIM % 4 == 0 && C % 4 == 0 && ((uintptr_t)a.qkv & 15) == 0) {       // 16-byte loads
      // every load of the chunk is issued before the first is stored (a loader's loads are all it waits for)
      constexpr int ITER = (CHUNK * (DIM / 4) + LOADERS - 1) / LOADERS > 0 ? (CHUNK * (DIM / 4) + LOADERS - 1) / LOADERS : 1;
      float4 qv[ITER], kv[ITER];
#pragma unroll
      for (int it = 0; it < ITER; ++it) {
        const int x = tid + it * nthreads;
        if (x < n * (DIM / 4)) {
          const int tt = x / (DIM / 4), d = 4 * (x - tt * (DIM / 4));
          const float* rowp = a.qkv + (size_t)(tc + tt) * C;
          qv[it] = *reinterpret_cast<const float4*>(rowp + g * DIM + d);
          kv[it] = *reinterpret_cast<const float4*>(rowp + GD + g * DIM + d);
        }
      }
#pragma unroll
      for (int it = 0; it < ITER; ++it) {
        const int x = tid + it * nthreads;
        if (x < n * (DIM / 4)) {
          const int tt = x / (DIM / 4), d = 4 * (x - tt * (DIM / 4));
          *reinterpret_cast<float4*>(&q_s[buf][tt][d]) = qv[it];
          *reinterpret_cast<float4*>(&k_s[buf][tt][d]) = kv[it];
        }
      }
    } else {
      for (int x = tid; x < n * DIM; x += nthreads) {
        const int tt = x / DIM, d = x - tt * DIM;
        const float* rowp = a.qkv + (size_t)(tc + tt) * C;
        q_s[buf][tt][d] = rowp[g * DIM + d];
        k_s[buf][tt][d] = rowp[GD + g * DIM + d];
      }
    }
    for (int x = tid; x < n * a.cols; x += nthreads) {
      const int tt = x / a.cols, cc = x - tt * a.cols;
      v_s[buf][tt][cc] = c0 + cc < a.V ? a.qkv[(size_t)(tc + tt) * C + 2 * GD + head * a.V + c0 + cc] : 0.f;
    }
    if (tid < n) {
      bg_s[buf][tid][0] = a.beta[(size_t)(tc + tid) * a.H + head];
      bg_s[buf][tid][1] = a.decay[(size_t)(tc + tid) * a.H + head];
    }
  };
  float* Sg = a.state + (size_t)slot * a.state_stride + a.s_off + (size_t)head * DIM * a.V;
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int d = i * R + r;
    S[i] = (live && d < DIM) ? Sg[(size_t)d * a.V + j] : 0.f;
  }
  fetch(0, t0, threadIdx.x, blockDim.x);
  __syncthreads();
  int buf = 0;
  for (int tc = t0; tc < t1; tc += CHUNK, buf ^= 1) {
    const int n = min(CHUNK, t1 - tc);
    if (loader) {
      if (tc + CHUNK < t1) fetch(buf ^ 1, tc + CHUNK, threadIdx.x - workers, LOADERS);
    } else {
#pragma unroll
      for (int tt = 0; tt < CHUNK; ++tt) {
        if (tt >= n) break;
        const float beta = bg_s[buf][tt][0], gd = bg_s[buf][tt][1];
        float kk[RPT];
        float dk = 0.f;
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          const int d = i * R + r;
          kk[i] = d < DIM ? k_s[buf][tt][d] : 0.f;
          S[i] *= gd;
          dk = fmaf(S[i], kk[i], dk);
        }
        dk = group_sum<R>(dk);
        const float u = beta * ((live ? v_s[buf][tt][col] : 0.f) - dk);
        float oq = 0.f;
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          const int d = i * R + r;
          S[i] = fmaf(kk[i], u, S[i]);
          oq = fmaf(S[i], d < DIM ? q_s[buf][tt][d] : 0.f, oq);
        }
        oq = group_sum<R>(oq);
        if (live && r == 0) a.o[(size_t)(tc + tt) * a.H * a.V + (size_t)head * a.V + j] = oq;
      }
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int d = i * R + r;
      if (d < DIM) Sg[(size_t)d * a.V + j] = S[i];
    }
  }
}

struct MlstmArgs {
  const void* proj;      // [T, ld] run dtype: q [H*DIM] | k [H*DIM] | v [H*V] | ...
  long long ld;
  const float* gates;    // [T, gld] fp32: zi [H] | zf [H]
  long long gld;
  const float* bi;       // [H]
  const float* bf;       // [H]
  float cap;
  float* state;          // per slot: S [H, DIM, V] at s_off, n [H, DIM] at n_off, m [H] at m_off
  long long state_stride, s_off, n_off, m_off;
  float* coef;           // [T, H, 3] fp32: e^(f+m-m'), e^(i-m'), the read-out's denominator
  float* o;              // [T, H*V] fp32
  int H, V, cols;
};

__device__ __forceinline__ float logsigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// The part of the recurrence that no column of S takes part in: the gates, the running maximum m,
// the normaliser n and the read-out's denominator.  One warp per (sequence, head) walks the tokens
// and leaves three numbers per token for the CTAs that own the columns; three more warps fetch the
// next tokens' q and k meanwhile and work out their gates' logarithms, which need no earlier token.
constexpr int NPL = (DIM + 31) / 32;          // entries of n per lane
constexpr int SCHUNK = DIM <= 64 ? 32 : DIM <= 128 ? 16 : DIM <= 256 ? 8 : DIM <= 512 ? 4 : 2;

template <typename T>
__global__ void __launch_bounds__(128) mlstm_scan_kernel(MlstmArgs a, IertBatchView b) {
  __shared__ __align__(16) float k_s[2][SCHUNK][DIM], q_s[2][SCHUNK][DIM], g_s[2][SCHUNK][2];
  pdl_wait();
  const int s = blockIdx.x, head = blockIdx.y, lane = threadIdx.x & 31;
  const int slot = b.slot_ids[s];
  const int t0 = b.cu_q[s], t1 = b.cu_q[s + 1];
  if (slot < 0 || t1 <= t0) return;
  const bool loader = threadIdx.x >= 32;
  const float qscale = 1.0f / sqrtf((float)DIM);
  const T* proj = (const T*)a.proj;
  auto fetch = [&](int buf, int tc, int tid, int nthreads) {
    const int n = min(SCHUNK, t1 - tc);
    if (sizeof(T) == 2 && DIM % 8 == 0 && a.ld % 8 == 0 && ((uintptr_t)a.proj & 15) == 0) {      // eight bf16 per load
      // every load of the chunk is issued before the first is converted and stored
      constexpr int ITER = (SCHUNK * (DIM / 8) * 2 + 96 - 1) / 96 > 0 ? (SCHUNK * (DIM / 8) * 2 + 96 - 1) / 96 : 1;     // key sizes below 8 never take this branch
      uint4 raw[ITER];
#pragma unroll
      for (int it = 0; it < ITER; ++it) {
        const int x = tid + it * nthreads;
        if (x < n * (DIM / 8) * 2) {
          const int which = x & 1, y = x >> 1;
          const int tt = y / (DIM / 8), d = 8 * (y - tt * (DIM / 8));
          raw[it] = *reinterpret_cast<const uint4*>(proj + (size_t)(tc + tt) * a.ld + (which ? a.H * DIM : 0) + head * DIM + d);
        }
      }
#pragma unroll
      for (int it = 0; it < ITER; ++it) {
        const int x = tid + it * nthreads;
        if (x < n * (DIM / 8) * 2) {
          const int which = x & 1, y = x >> 1;
          const int tt = y / (DIM / 8), d = 8 * (y - tt * (DIM / 8));
          const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw[it]);
          float* dst = which ? &k_s[buf][tt][d] : &q_s[buf][tt][d];
          const float sc = which ? 1.f : qscale;
          const float2 f0 = __bfloat1622float2(p[0]), f1 = __bfloat1622float2(p[1]);
          const float2 f2 = __bfloat1622float2(p[2]), f3 = __bfloat1622float2(p[3]);
          *reinterpret_cast<float4*>(dst) = make_float4(f0.x * sc, f0.y * sc, f1.x * sc, f1.y * sc);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(f2.x * sc, f2.y * sc, f3.x * sc, f3.y * sc);
        }
      }
    } else {
      for (int x = tid; x < n * DIM; x += nthreads) {
        const int tt = x / DIM, d = x - tt * DIM;
        const T* rowp = proj + (size_t)(tc + tt) * a.ld;
        q_s[buf][tt][d] = to_f32(rowp[head * DIM + d]) * qscale;
        k_s[buf][tt][d] = to_f32(rowp[a.H * DIM + head * DIM + d]);
      }
    }
    for (int tt = tid; tt < n; tt += nthreads) {
      const float zi = a.gates[(size_t)(tc + tt) * a.gld + head] + a.bi[head];
      const float zf = a.gates[(size_t)(tc + tt) * a.gld + a.H + head] + a.bf[head];
      g_s[buf][tt][0] = a.cap * tanhf(zi / a.cap);
      g_s[buf][tt][1] = logsigmoid_f(a.cap * tanhf(zf / a.cap));
    }
  };
  float* base = a.state + (size_t)slot * a.state_stride;
  float* ng = base + a.n_off + (size_t)head * DIM;
  float nn[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) nn[i] = lane + 32 * i < DIM ? ng[lane + 32 * i] : 0.f;
  float m = base[a.m_off + head];
  fetch(0, t0, threadIdx.x, blockDim.x);
  __syncthreads();
  int buf = 0;
  for (int tc = t0; tc < t1; tc += SCHUNK, buf ^= 1) {
    const int n = min(SCHUNK, t1 - tc);
    if (loader) {
      if (tc + SCHUNK < t1) fetch(buf ^ 1, tc + SCHUNK, threadIdx.x - 32, blockDim.x - 32);
    } else {
#pragma unroll 4
      for (int tt = 0; tt < SCHUNK; ++tt) {
        if (tt >= n) break;
        const float li = g_s[buf][tt][0], lf = g_s[buf][tt][1];
        const float m_new = fmaxf(lf + m, li);
        const float ea = expf(lf + m - m_new), eb = expf(li - m_new);
        m = m_new;
        float nq = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          const int d = lane + 32 * i;
          if (d < DIM) {
            nn[i] = fmaf(ea, nn[i], eb * k_s[buf][tt][d]);
            nq = fmaf(nn[i], q_s[buf][tt][d], nq);
          }
        }
        nq = warp_sum(nq);
        if (lane == 0) {
          float* c = a.coef + ((size_t)(tc + tt) * a.H + head) * 3;
          c[0] = ea; c[1] = eb; c[2] = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
        }
      }
    }
    __syncthreads();
  }
  if (!loader) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) if (lane + 32 * i < DIM) ng[lane + 32 * i] = nn[i];
    if (lane == 0) base[a.m_off + head] = m;
  }
}

template <typename T, int R>
__global__ void __launch_bounds__(256 + LOADERS) mlstm_recur_kernel(MlstmArgs a, IertBatchView b) {
  constexpr int RPT = (DIM + R - 1) / R;
  __shared__ __align__(16) float k_s[2][CHUNK][DIM], q_s[2][CHUNK][DIM], v_s[2][CHUNK][256], c_s[2][CHUNK][3];
  pdl_wait();
  const int s = blockIdx.x, head = blockIdx.y, c0 = blockIdx.z * a.cols;
  const int slot = b.slot_ids[s];
  const int t0 = b.cu_q[s], t1 = b.cu_q[s + 1];
  if (slot < 0 || t1 <= t0) return;
  const int workers = blockDim.x - LOADERS;
  const bool loader = (int)threadIdx.x >= workers;
  const int col = threadIdx.x / R, r = threadIdx.x % R;
  const int j = c0 + col;
  const bool live = !loader && col < a.cols && j < a.V;
  const float qscale = 1.0f / sqrtf((float)DIM);
  const T* proj = (const T*)a.proj;
  auto fetch = [&](int buf, int tc, int tid, int nthreads) {
    const int n = min(CHUNK, t1 - tc);
    if (sizeof(T) == 2 && DIM % 8 == 0 && a.ld % 8 == 0 && ((uintptr_t)a.proj & 15) == 0) {      // eight bf16 per load
      // every load of the chunk is issued before the first is converted and stored
      constexpr int ITER = (CHUNK * (DIM / 8) * 2 + LOADERS - 1) / LOADERS > 0 ? (CHUNK * (DIM / 8) * 2 + LOADERS - 1) / LOADERS : 1;
      uint4 raw[ITER];
#pragma unroll
      for (int it = 0; it < ITER; ++it) {
        const int x = tid + it * nthreads;
        if (x < n * (DIM / 8) * 2) {
          const int which = x & 1, y = x >> 1;
          const int tt = y / (DIM / 8), d = 8 * (y - tt * (DIM / 8));
          raw[it] = *reinterpret_cast<const uint4*>(proj + (size_t)(tc + tt) * a.ld + (which ? a.H * DIM : 0) + head * DIM + d);
        }
      }
#pragma unroll
      for (int it = 0; it < ITER; ++it) {
        const int x = tid + it * nthreads;
        if (x < n * (DIM / 8) * 2) {
          const int which = x & 1, y = x >> 1;
          const int tt = y / (DIM / 8), d = 8 * (y - tt * (DIM / 8));
          const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw[it]);
          float* dst = which ? &k_s[buf][tt][d] : &q_s[buf][tt][d];
          const float sc = which ? 1.f : qscale;
          const float2 f0 = __bfloat1622float2(p[0]), f1 = __bfloat1622float2(p[1]);
          const float2 f2 = __bfloat1622float2(p[2]), f3 = __bfloat1622float2(p[3]);
          *reinterpret_cast<float4*>(dst) = make_float4(f0.x * sc, f0.y * sc, f1.x * sc, f1.y * sc);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(f2.x * sc, f2.y * sc, f3.x * sc, f3.y * sc);
        }
      }
    } else {
      for (int x = tid; x < n * DIM; x += nthreads) {
        const int tt = x / DIM, d = x - tt * DIM;
        const T* rowp = proj + (size_t)(tc + tt) * a.ld;
        q_s[buf][tt][d] = to_f32(rowp[head * DIM + d]) * qscale;
        k_s[buf][tt][d] = to_f32(rowp[a.H * DIM + head * DIM + d]);
      }
    }
    for (int x = tid; x < n * a.cols; x += nthreads) {
      const int tt = x / a.cols, cc = x - tt * a.cols;
      v_s[buf][tt][cc] = c0 + cc < a.V ? to_f32(proj[(size_t)(tc + tt) * a.ld + 2 * a.H * DIM + head * a.V + c0 + cc]) : 0.f;
    }
    if (tid < n * 3) c_s[buf][tid / 3][tid % 3] = a.coef[((size_t)(tc + tid / 3) * a.H + head) * 3 + tid % 3];
  };
  float* Sg = a.state + (size_t)slot * a.state_stride + a.s_off + (size_t)head * DIM * a.V;
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int d = i * R + r;
    S[i] = (live && d < DIM) ? Sg[(size_t)d * a.V + j] : 0.f;
  }
  fetch(0, t0, threadIdx.x, blockDim.x);
  __syncthreads();
  int buf = 0;
  for (int tc = t0; tc < t1; tc += CHUNK, buf ^= 1) {
    const int n = min(CHUNK, t1 - tc);
    if (loader) {
      if (tc + CHUNK < t1) fetch(buf ^ 1, tc + CHUNK, threadIdx.x - workers, LOADERS);
    } else {
#pragma unroll
      for (int tt = 0; tt < CHUNK; ++tt) {
        if (tt >= n) break;
        const float ea = c_s[buf][tt][0], eb = c_s[buf][tt][1], den = c_s[buf][tt][2];
        const float bv = eb * (live ? v_s[buf][tt][col] : 0.f);
        float oq = 0.f;
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          const int d = i * R + r;
          const float kd = d < DIM ? k_s[buf][tt][d] : 0.f, qd = d < DIM ? q_s[buf][tt][d] : 0.f;
          S[i] = fmaf(ea, S[i], kd * bv);
          oq = fmaf(S[i], qd, oq);
        }
        oq = group_sum<R>(oq);
        if (live && r == 0) a.o[(size_t)(tc + tt) * a.H * a.V + (size_t)head * a.V + j] = oq / den;
      }
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int d = i * R + r;
      if (d < DIM) Sg[(size_t)d * a.V + j] = S[i];
    }
  }
}

struct WkvArgs {
  const float* x;        // [T, ld] fp32: r [H*DIM] | k [H*DIM] | v [H*V] | ... (the projections)
  long long ld;
  const float* decay;    // [T, H*DIM] fp32: w, the factor of each row of S
  const float* u;        // [H, DIM] fp32: the current token's bonus
  float* state;          // per slot at s_off: S [H, DIM, V]
  long long state_stride, s_off;
  float* o;              // [T, H*V] fp32
  int H, V, cols;
};

template <int R>
__global__ void __launch_bounds__(256 + LOADERS) wkv_recur_kernel(WkvArgs a, IertBatchView b) {
  constexpr int RPT = (DIM + R - 1) / R;
  __shared__ __align__(16) float r_s[2][CHUNK][DIM], k_s[2][CHUNK][DIM], w_s[2][CHUNK][DIM], v_s[2][CHUNK][256];
  pdl_wait();
  const int s = blockIdx.x, head = blockIdx.y, c0 = blockIdx.z * a.cols;
  const int slot = b.slot_ids[s];
  const int t0 = b.cu_q[s], t1 = b.cu_q[s + 1];
  if (slot < 0 || t1 <= t0) return;
  const int workers = blockDim.x - LOADERS;
  const bool loader = (int)threadIdx.x >= workers;
  const int col = threadIdx.x / R, r = threadIdx.x % R;
  const int j = c0 + col;
  const bool live = !loader && col < a.cols && j < a.V;
  const int HD = a.H * DIM;
  auto fetch = [&](int buf, int tc, int tid, int nthreads) {
    const int n = min(CHUNK, t1 - tc);
    if (DIM % 4 == 0 && a.ld % 4 == 0 && ((uintptr_t)a.x & 15) == 0 && ((uintptr_t)a.decay & 15) == 0) {     // 16-byte loads
      // every load of the chunk is issued before the first is stored (a loader's loads are all it waits for)
      constexpr int ITER = (CHUNK * (DIM / 4) + LOADERS - 1) / LOADERS > 0 ? (CHUNK * (DIM / 4) + LOADERS - 1) / LOADERS : 1;
      float4 rv[ITER], kv[ITER], wv[ITER];
#pragma unroll
      for (int it = 0; it < ITER; ++it) {
        const int x = tid + it * nthreads;
        if (x < n * (DIM / 4)) {
          const int tt = x / (DIM / 4), d = 4 * (x - tt * (DIM / 4));
          const float* rowp = a.x + (size_t)(tc + tt) * a.ld + head * DIM + d;
          rv[it] = *reinterpret_cast<const float4*>(rowp);
          kv[it] = *reinterpret_cast<const float4*>(rowp + HD);
          wv[it] = *reinterpret_cast<const float4*>(a.decay + (size_t)(tc + tt) * HD + head * DIM + d);
        }
      }
#pragma unroll
      for (int it = 0; it < ITER; ++it) {
        const int x = tid + it * nthreads;
        if (x < n * (DIM / 4)) {
          const int tt = x / (DIM / 4), d = 4 * (x - tt * (DIM / 4));
          *reinterpret_cast<float4*>(&r_s[buf][tt][d]) = rv[it];
          *reinterpret_cast<float4*>(&k_s[buf][tt][d]) = kv[it];
          *reinterpret_cast<float4*>(&w_s[buf][tt][d]) = wv[it];
        }
      }
    } else {
      for (int x = tid; x < n * DIM; x += nthreads) {
        const int tt = x / DIM, d = x - tt * DIM;
        const float* rowp = a.x + (size_t)(tc + tt) * a.ld + head * DIM + d;
        r_s[buf][tt][d] = rowp[0];
        k_s[buf][tt][d] = rowp[HD];
        w_s[buf][tt][d] = a.decay[(size_t)(tc + tt) * HD + head * DIM + d];
      }
    }
    for (int x = tid; x < n * a.cols; x += nthreads) {
      const int tt = x / a.cols, cc = x - tt * a.cols;
      v_s[buf][tt][cc] = c0 + cc < a.V ? a.x[(size_t)(tc + tt) * a.ld + 2 * HD + head * a.V + c0 + cc] : 0.f;
    }
  };
  float* Sg = a.state + (size_t)slot * a.state_stride + a.s_off + (size_t)head * DIM * a.V;
  float S[RPT], u[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int d = i * R + r;
    S[i] = (live && d < DIM) ? Sg[(size_t)d * a.V + j] : 0.f;
    u[i] = d < DIM ? a.u[head * DIM + d] : 0.f;
  }
  fetch(0, t0, threadIdx.x, blockDim.x);
  __syncthreads();
  int buf = 0;
  for (int tc = t0; tc < t1; tc += CHUNK, buf ^= 1) {
    const int n = min(CHUNK, t1 - tc);
    if (loader) {
      if (tc + CHUNK < t1) fetch(buf ^ 1, tc + CHUNK, threadIdx.x - workers, LOADERS);
    } else {
#pragma unroll
      for (int tt = 0; tt < CHUNK; ++tt) {
        if (tt >= n) break;
        const float vj = live ? v_s[buf][tt][col] : 0.f;
        float oq = 0.f;
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          const int d = i * R + r;
          const float kd = d < DIM ? k_s[buf][tt][d] : 0.f, rd = d < DIM ? r_s[buf][tt][d] : 0.f;
          const float wd = d < DIM ? w_s[buf][tt][d] : 0.f;
          const float kv = kd * vj;
          oq = fmaf(rd, fmaf(u[i], kv, S[i]), oq);
          S[i] = fmaf(wd, S[i], kv);
        }
        oq = group_sum<R>(oq);
        if (live && r == 0) a.o[(size_t)(tc + tt) * a.H * a.V + (size_t)head * a.V + j] = oq;
      }
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int d = i * R + r;
      if (d < DIM) Sg[(size_t)d * a.V + j] = S[i];
    }
  }
}

// Lanes per column: the fewest that give the device about eight warps per SM (at most 32), and columns per
// CTA so that a CTA has up to 256 computing threads.  (Measured at 32 heads of 128 x 128, one prompt of 2,048
// tokens: 8 lanes per column 1.08 ms, 16 lanes 0.91 ms, 32 lanes 1.42 ms per layer.)
struct Split { int lanes, cols; };
Split pick_split(int n_seqs, int H, int V) {
  const long long want = 8LL * 32 * iert_sm_count_cached();          // threads
  int lanes = R_MIN;
  while (lanes < 32 && (long long)n_seqs * H * V * lanes < want) lanes *= 2;
  if (const char* forced = getenv("IERT_RECURRENT_LANES")) {         // for tests and measurements: 1, 2, ... 32
    const int f = atoi(forced);
    if (f >= 1) { lanes = R_MIN; while (lanes < 32 && lanes < f) lanes *= 2; }
  }
  int cols = 256 / lanes;
  if (cols > V) cols = V;
  return {lanes, cols};
}

}  // namespace

IERT_API int iert_recurrent_dim() { return DIM; }

#define IERT_BY_LANES(L, CALL)                                       \
  switch (L) {                                                       \
    case 1: { constexpr int RR = 1 < R_MIN ? R_MIN : 1; CALL; } break;    \
    case 2: { constexpr int RR = 2 < R_MIN ? R_MIN : 2; CALL; } break;    \
    case 4: { constexpr int RR = 4 < R_MIN ? R_MIN : 4; CALL; } break;    \
    case 8: { constexpr int RR = 8 < R_MIN ? R_MIN : 8; CALL; } break;    \
    case 16: { constexpr int RR = 16 < R_MIN ? R_MIN : 16; CALL; } break; \
    default: { constexpr int RR = 32; CALL; } break;                 \
  }

IERT_API int iert_delta_recur(const float* qkv, const float* beta, const float* decay, float* state,
                              long long state_stride, long long s_off, float* o, int G, int H, int V,
                              const IertBatchView* batch, cudaStream_t stream) {
  if (batch->n_seqs <= 0 || batch->n_tokens <= 0) return IERT_OK;
  if (G <= 0 || H <= 0 || H % G || V <= 0 || H > 65535) return IERT_BAD_ARGUMENT;
  const Split sp = pick_split(batch->n_seqs, H, V);
  DeltaArgs a = {qkv, beta, decay, state, state_stride, s_off, o, G, H, V, sp.cols};
  dim3 grid(batch->n_seqs, H, (V + sp.cols - 1) / sp.cols);
  const int threads = ((sp.cols * sp.lanes + 31) / 32) * 32 + LOADERS;
  IERT_BY_LANES(sp.lanes, launch_dep(delta_recur_kernel<RR>, grid, dim3(threads), 0, stream, a, *batch));
  return iert_check_launch("delta_recur");
}

// x: fp32 [T, ld] = r [H*DIM] | k [H*DIM] | v [H*V] | ...; decay fp32 [T, H*DIM]; u fp32 [H, DIM]; o fp32 [T, H*V].
IERT_API int iert_wkv_recur(const float* x, long long ld, const float* decay, const float* u, float* state,
                            long long state_stride, long long s_off, float* o, int H, int V, const IertBatchView* batch,
                            cudaStream_t stream) {
  if (batch->n_seqs <= 0 || batch->n_tokens <= 0) return IERT_OK;
  if (H <= 0 || V <= 0 || H > 65535 || ld < (long long)2 * H * DIM + (long long)H * V) return IERT_BAD_ARGUMENT;
  const Split sp = pick_split(batch->n_seqs, H, V);
  WkvArgs a = {x, ld, decay, u, state, state_stride, s_off, o, H, V, sp.cols};
  dim3 grid(batch->n_seqs, H, (V + sp.cols - 1) / sp.cols);
  const int threads = ((sp.cols * sp.lanes + 31) / 32) * 32 + LOADERS;
  IERT_BY_LANES(sp.lanes, launch_dep(wkv_recur_kernel<RR>, grid, dim3(threads), 0, stream, a, *batch));
  return iert_check_launch("wkv_recur");
}

IERT_API int iert_mlstm_recur(const void* proj, int dtype, long long ld, const float* gates, long long gld,
                              const float* bi, const float* bf, float cap, float* state, long long state_stride,
                              long long s_off, long long n_off, long long m_off, float* coef, float* o, int H, int V,
                              const IertBatchView* batch, cudaStream_t stream) {
  if (batch->n_seqs <= 0 || batch->n_tokens <= 0) return IERT_OK;
  if (H <= 0 || V <= 0 || H > 65535 || !(cap > 0.f) || (dtype != IERT_F32 && dtype != IERT_BF16)) return IERT_BAD_ARGUMENT;
  const Split sp = pick_split(batch->n_seqs, H, V);
  MlstmArgs a = {proj, ld, gates, gld, bi, bf, cap, state, state_stride, s_off, n_off, m_off, coef, o, H, V, sp.cols};
  dim3 grid(batch->n_seqs, H, (V + sp.cols - 1) / sp.cols);
  const int threads = ((sp.cols * sp.lanes + 31) / 32) * 32 + LOADERS;
  if (dtype == IERT_F32) {
    launch_dep(mlstm_scan_kernel<float>, dim3(batch->n_seqs, H), dim3(128), 0, stream, a, *batch);
    IERT_BY_LANES(sp.lanes, (launch_dep(mlstm_recur_kernel<float, RR>, grid, dim3(threads), 0, stream, a, *batch)));
  } else {
    launch_dep(mlstm_scan_kernel<__nv_bfloat16>, dim3(batch->n_seqs, H), dim3(128), 0, stream, a, *batch);
    IERT_BY_LANES(sp.lanes, (launch_dep(mlstm_recur_kernel<__nv_bfloat16, RR>, grid, dim3(threads), 0, stream, a, *batch)));
  }
  return iert_check_launch("mlstm_recur");
}
