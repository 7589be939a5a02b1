// Routing of a mixture-of-experts feed-forward.
//
// router_topk: logits z = x W_r^T (+ bias) arrive in fp32 [T, E]; the `top` largest are chosen (the
//   lower index wins a tie) and their weights are the softmax over the chosen logits only.  Written as
//   a dense map wt [T, E] (zero for experts not chosen) and as lists idx / w [T, top].
// router_grouped: the logits cover N = E + I outputs, the last I of which stand for experts that return their
//   input.  Scores s = softmax(z) over all N; the choice is made on s + correction: the N outputs form `groups`
//   equal runs of neighbours, a group's score is its largest choice score, only members of the `keep` best groups
//   can be chosen (the others count as minus infinity), and of those the `top` largest are (the lower index wins a
//   tie everywhere).  The weights are the chosen s divided by their sum (+ 1e-20).  Written as a dense map
//   wt [T, E] over the experts with tensors, as wid [T] (the sum of the weights of chosen identity experts) and
//   as lists idx / w [T, top].
// moe_scale: act[t, e*F + i] *= wt[t, e] for the E routed experts' blocks of F activations; columns
//   beyond E*F (an expert that every token uses) are left as they are.  With `wid`: also
//   residual[t, :] += wid[t] * x[t, :] (the identity experts' share; x in the activations' dtype).
#include "common.cuh"

using namespace iert;

namespace {

constexpr int MAX_TOP = 32;

__global__ void router_topk_kernel(const float* __restrict__ z, long long ldz, const float* __restrict__ bias,
                                   int E, int top, float* __restrict__ wt, int* __restrict__ idx,
                                   float* __restrict__ w) {
  // one warp per token
  pdl_launch_dependents();     // the next kernel may start its preamble now
  pdl_wait();                  // everything below may depend on the kernel before
  const int t = blockIdx.x, lane = threadIdx.x;
  const float* row = z + (size_t)t * ldz;
  int chosen[MAX_TOP];
  float val[MAX_TOP];
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= chosen[j] == e;
      const float v = row[e] + (bias ? bias[e] : 0.f);
      if (!taken && (v > best || (v == best && e < bi))) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    chosen[k] = bi;
    val[k] = best;
  }
  float den = 0.f;
  const float largest = val[0];
  for (int k = 0; k < top; ++k) { val[k] = expf(val[k] - largest); den += val[k]; }
  for (int e = lane; e < E; e += 32) wt[(size_t)t * E + e] = 0.f;
  __syncwarp();
  if (lane == 0)
    for (int k = 0; k < top; ++k) {
      const float p = val[k] / den;
      if (chosen[k] < E) wt[(size_t)t * E + chosen[k]] = p;
      idx[(size_t)t * top + k] = chosen[k];
      w[(size_t)t * top + k] = p;
    }
}

// one warp per token; shared memory: s[N], c[N], group score [groups], flags [N] (bytes).  Output e of token t is
// z[t * ldz + e * lde]: rows of tokens (lde = 1) or rows of outputs (ldz = 1).
//   score_mode   0: scores are the softmax over all N outputs; 1: every output's own sigmoid
//   group_mode   0: a group's score is its best choice score; 1: the sum of its two best (of its one, if it has one)
//   weights      chosen scores / (their sum + weight_eps) * weight_scale
__global__ void router_grouped_kernel(const float* __restrict__ z, long long ldz, long long lde, const float* __restrict__ correction, int E,
                                      int N, int top, int groups, int keep, int score_mode, int group_mode, float weight_eps,
                                      float weight_scale, float* __restrict__ wt, float* __restrict__ wid,
                                      int* __restrict__ idx, float* __restrict__ w) {
  extern __shared__ float rsm[];
  float* s = rsm;
  float* c = rsm + N;
  float* gs = rsm + 2 * N;
  unsigned char* open = reinterpret_cast<unsigned char*>(rsm + 2 * N + groups);      // 1: may still be chosen
  pdl_launch_dependents();     // the next kernel (the experts' product) may fetch its first weights now
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x, per = N / groups;
  const float* row = z + (size_t)t * ldz;
  float den = 1.f;
  if (score_mode == 0) {
    float m = -INFINITY;
    for (int e = lane; e < N; e += 32) m = fmaxf(m, row[e * lde]);
    m = warp_max(m);
    den = 0.f;
    for (int e = lane; e < N; e += 32) { const float p = expf(row[e * lde] - m); s[e] = p; den += p; }
    den = warp_sum(den);
  } else {
    for (int e = lane; e < N; e += 32) s[e] = 1.0f / (1.0f + expf(-row[e * lde]));
  }
  for (int e = lane; e < N; e += 32) {
    s[e] = s[e] / den;
    c[e] = s[e] + (correction ? correction[e] : 0.f);
    open[e] = 0;
  }
  __syncwarp();
  for (int g = lane; g < groups; g += 32) {
    float best = -INFINITY, second = -INFINITY;
    for (int j = 0; j < per; ++j) {
      const float v = c[g * per + j];
      if (v > best) { second = best; best = v; }
      else if (v > second) second = v;
    }
    gs[g] = group_mode == 1 && per > 1 ? best + second : best;
  }
  __syncwarp();
  // the `keep` best groups, one after the other; a group that was taken is marked by NaN
  for (int k = 0; k < keep; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int g = lane; g < groups; g += 32) {
      const float v = gs[g];
      if (v == v && (v > best || (v == best && g < bi) || bi == 0x7fffffff)) { best = v; bi = g; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
    }
    __syncwarp();
    if (bi != 0x7fffffff) {
      for (int j = lane; j < per; j += 32) open[bi * per + j] = 1;
      if (lane == 0) gs[bi] = __int_as_float(0x7fc00000);
    }
    __syncwarp();
  }
  int chosen[MAX_TOP];
  float val[MAX_TOP];
  float sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < N; e += 32) {
      const float v = c[e];
      if (open[e] && (bi == 0x7fffffff || v > best || (v == best && e < bi))) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
    }
    __syncwarp();
    chosen[k] = bi;
    val[k] = bi != 0x7fffffff ? s[bi] : 0.f;
    sum += val[k];
    if (lane == 0 && bi != 0x7fffffff) open[bi] = 0;
    __syncwarp();
  }
  for (int e = lane; e < E; e += 32) wt[(size_t)t * E + e] = 0.f;
  __syncwarp();
  if (lane == 0) {
    float identity = 0.f;
    for (int k = 0; k < top; ++k) {
      const float p = val[k] / (sum + weight_eps) * weight_scale;
      if (chosen[k] < E) wt[(size_t)t * E + chosen[k]] = p;
      else if (chosen[k] < N) identity += p;
      idx[(size_t)t * top + k] = chosen[k] < N ? chosen[k] : -1;
      w[(size_t)t * top + k] = p;
    }
    wid[t] = identity;
  }
}

template <typename T>
__global__ void moe_scale_kernel(T* __restrict__ act, long long ld, const float* __restrict__ wt, int E, int F,
                                 const float* __restrict__ wid, const T* __restrict__ x, long long ldx,
                                 float* __restrict__ residual, int H) {
  pdl_launch_dependents();     // the down product may fetch its first weights now
  pdl_wait();
  const int t = blockIdx.x;
  T* row = act + (size_t)t * ld;
  if (wid) {
    const float a = wid[t];
    if (a != 0.f)
      for (int i = threadIdx.x; i < H; i += blockDim.x) residual[(size_t)t * H + i] += a * to_f32(x[(size_t)t * ldx + i]);
  }
  if (sizeof(T) == 2 && F % 8 == 0 && ld % 8 == 0 && ((uintptr_t)act & 15) == 0) {      // eight at a time
    for (int i = threadIdx.x * 8; i < E * F; i += blockDim.x * 8) {
      const float w = wt[(size_t)t * E + i / F];
      uint4 v = *reinterpret_cast<const uint4*>(row + i);
      __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p[e]);
        p[e] = __floats2bfloat162_rn(f.x * w, f.y * w);
      }
      *reinterpret_cast<uint4*>(row + i) = v;
    }
    return;
  }
  for (int i = threadIdx.x; i < E * F; i += blockDim.x)
    row[i] = from_f32<T>(to_f32(row[i]) * wt[(size_t)t * E + i / F]);
}

}  // namespace

IERT_API int iert_router_topk(const float* z, long long ldz, const float* bias, int n_tokens, int E, int top,
                              float* wt, int* idx, float* w, cudaStream_t stream) {
  if (n_tokens <= 0) return IERT_OK;
  if (E <= 0 || top <= 0 || top > E || top > MAX_TOP) return IERT_BAD_ARGUMENT;
  launch_dep(router_topk_kernel, dim3(n_tokens), dim3(32), 0, stream, z, ldz, bias, E, top, wt, idx, w);
  return iert_check_launch("router_topk");
}

// z: output e of token t at z[t * ldz + e * lde] (fp32).
IERT_API int iert_router_grouped(const float* z, long long ldz, long long lde, const float* correction, int n_tokens, int E, int N, int top,
                                 int groups, int keep, int score_mode, int group_mode, float weight_eps, float weight_scale,
                                 float* wt, float* wid, int* idx, float* w, cudaStream_t stream) {
  if (n_tokens <= 0) return IERT_OK;
  if (score_mode < 0 || score_mode > 1 || group_mode < 0 || group_mode > 1) return IERT_BAD_ARGUMENT;
  if (E < 0 || N < E || N <= 0 || top <= 0 || top > MAX_TOP || groups <= 0 || N % groups || keep <= 0 || keep > groups ||
      top > keep * (N / groups))
    return IERT_BAD_ARGUMENT;
  const size_t smem = (size_t)(2 * N + groups) * sizeof(float) + (size_t)N;
  if (smem > 48 * 1024) return IERT_BAD_ARGUMENT;
  launch_dep(router_grouped_kernel, dim3(n_tokens), dim3(32), smem, stream, z, ldz, lde, correction, E, N, top, groups, keep, score_mode,
             group_mode, weight_eps, weight_scale, wt, wid, idx, w);
  return iert_check_launch("router_grouped");
}

// wid (optional, fp32 [T]) with x ([T, H], stride ldx, the activations' dtype) and residual (fp32 [T, H]): the share of
// experts that return their input.
IERT_API int iert_moe_scale(void* act, int dtype, long long ld, const float* wt, int n_tokens, int E, int F, const float* wid,
                            const void* x, long long ldx, float* residual, int H, cudaStream_t stream) {
  if (n_tokens <= 0) return IERT_OK;
  if (E < 0 || F <= 0 || (wid && (!x || !residual || H <= 0))) return IERT_BAD_ARGUMENT;
  if (dtype == IERT_F32)
    launch_dep(moe_scale_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, (float*)act, ld, wt, E, F, wid, (const float*)x, ldx,
               residual, H);
  else if (dtype == IERT_BF16)
    launch_dep(moe_scale_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, stream, (__nv_bfloat16*)act, ld, wt, E, F, wid,
               (const __nv_bfloat16*)x, ldx, residual, H);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("moe_scale");
}
