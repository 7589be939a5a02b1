// One-token steps of latent attention on the tensor cores (mma.sync m16n8k16, bf16 in, fp32 out),
// in the absorbed form: every head's query is first taken into the latent's coordinates,
// qa = W_uk[h]^T q (rank numbers), so that all heads of a sequence meet the same cached rows c_j:
//
//   S = Qa C^T   ([heads x rank] x [rank x keys]),   P = softmax with a sink,   L = P C  ([heads x keys] x [keys x rank])
//
// which is multi-query attention whose keys and values are the same rows.  W_uv is applied to L at the
// end, once per head.  Three kernels:
//   latent_absorb_q       qa [T, Hpad, rank] bf16 from q and W_uk (rows of padding heads are zero)
//   latent_decode_tc      a CTA takes (sequence, a run of 64-key tiles, up to 32 heads): the tile of C comes
//                         into shared memory once (cp.async) and serves both products; warp w forms the
//                         scores of keys 16w..16w+15 of the tile for all the CTA's heads, the warps agree on
//                         row maxima and sums through shared memory, and warp w then owns a quarter of the
//                         rank columns of L (its accumulators).  Partial (max, sum, L) per run go to scratch.
//   latent_decode_merge   merges the runs in order, adds the sink's term exp(sink - M) to the denominator,
//                         and multiplies by W_uv: out [T, H*V].
// Sizes: rank a multiple of 32 up to 512, pages of 64 positions, a bf16 cache.  Anything else is refused
// (IERT_BAD_ARGUMENT) and the caller runs the plain kernel.
#include "common.cuh"

using namespace iert;

namespace {

constexpr int BK = 64;            // keys per tile = positions per page
constexpr int THREADS = 128;
constexpr int MAX_NTW = 16;       // n-tiles of 8 rank columns per warp: rank <= 4 * 16 * 8 = 512
constexpr int PLD = BK + 8;       // row stride of the probabilities in shared memory (elements)

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t lds32(const __nv_bfloat16* p) { return *reinterpret_cast<const uint32_t*>(p); }

// qa[t, h, :] = sum_d q[t, h, d] W_uk[h*D + d, :].  A block of 256 threads takes one (token, head): 64 threads
// across the rank (eight columns each, 16-byte loads of the weights) times four groups along d, added
// through shared memory in a fixed order.
constexpr int ABSORB_THREADS = 256;

__global__ void __launch_bounds__(ABSORB_THREADS)
latent_absorb_q_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const __nv_bfloat16* __restrict__ w_uk,
                       __nv_bfloat16* __restrict__ qa, int H, int Hpad, int D, int R, int rank) {
  extern __shared__ float sm_q[];
  float* q_s = sm_q;                    // [D]
  float* part = sm_q + D;               // [4][rank]
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  __nv_bfloat16* dst = qa + ((size_t)t * Hpad + h) * (rank + R);
  if (h >= H) {
    for (int r = threadIdx.x; r < rank + R; r += blockDim.x) dst[r] = __float2bfloat16_rn(0.f);
    return;
  }
  const __nv_bfloat16* qh = q + (size_t)t * ldq + (size_t)h * (D + R);
  for (int d = threadIdx.x; d < D; d += blockDim.x) q_s[d] = __bfloat162float(qh[d]);
  for (int i = threadIdx.x; i < R; i += blockDim.x) dst[rank + i] = qh[D + i];      // the rotated part passes as it is
  __syncthreads();
  const int grp = threadIdx.x >> 6, lane64 = threadIdx.x & 63;
  const int d_lo = grp * ((D + 3) / 4), d_hi = min(D, d_lo + (D + 3) / 4);
  for (int r0 = lane64 * 8; r0 < rank; r0 += 64 * 8) {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const __nv_bfloat16* w = w_uk + (size_t)h * D * rank + r0;
#pragma unroll 4
    for (int d = d_lo; d < d_hi; ++d) {
      const uint4 v = *reinterpret_cast<const uint4*>(w + (size_t)d * rank);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
      const float qd = q_s[d];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p[e]);
        a[2 * e] = fmaf(qd, f.x, a[2 * e]);
        a[2 * e + 1] = fmaf(qd, f.y, a[2 * e + 1]);
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) part[grp * rank + r0 + e] = a[e];
  }
  __syncthreads();
  for (int r = threadIdx.x; r < rank; r += blockDim.x)
    dst[r] = __float2bfloat16_rn((part[r] + part[rank + r]) + (part[2 * rank + r] + part[3 * rank + r]));
}

template <int MT>
__global__ void __launch_bounds__(THREADS)
latent_decode_tc_kernel(const __nv_bfloat16* __restrict__ qa, IertBatchView b, IertKvView kv, int Hpad, int R, float scale,
                        int splits, float* __restrict__ part_m, float* __restrict__ part_l,
                        float* __restrict__ part_acc, int* __restrict__ err) {
  extern __shared__ __align__(16) uint8_t smem[];
  // a cached row is `width` numbers: the latent (`rank`, which also serves as the value) and R rotated key numbers
  const int width = kv.head_dim, rank = width - R, ldc = width + 8;
  __nv_bfloat16* qa_s = reinterpret_cast<__nv_bfloat16*>(smem);     // [MT*16][ldc]
  __nv_bfloat16* c_s = qa_s + MT * 16 * ldc;                         // [BK][ldc]
  __nv_bfloat16* p_s = c_s + BK * ldc;                               // [MT*16][PLD]
  float* wmax = reinterpret_cast<float*>(p_s + MT * 16 * PLD);       // [4][MT*16]
  float* wsum = wmax + 4 * MT * 16;                                  // [4][MT*16]
  pdl_wait();
  const int s = blockIdx.x, split = blockIdx.y, rows0 = blockIdx.z * MT * 16;
  const int slot = b.slot_ids[s];
  if (slot < 0) return;
  const int n_keys = b.pos0[s] + 1;                  // one token per sequence: its own row is in the cache
  const int n_tiles = (n_keys + BK - 1) / BK;
  const int t_lo = (int)((long long)split * n_tiles / splits), t_hi = (int)((long long)(split + 1) * n_tiles / splits);
  const size_t part_row0 = ((size_t)s * splits + split) * Hpad + rows0;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  if (t_lo >= t_hi) {                                // an empty run: a partial that the merge skips
    if (tid < MT * 16) { part_m[part_row0 + tid] = -INFINITY; part_l[part_row0 + tid] = 0.f; }
    return;
  }
  const int chunks = width / 8;                      // 16-byte pieces per row
  for (int i = tid; i < MT * 16 * chunks; i += THREADS) {
    const int r = i / chunks, c = i - r * chunks;
    *reinterpret_cast<uint4*>(qa_s + r * ldc + c * 8) =
        *reinterpret_cast<const uint4*>(qa + ((size_t)s * Hpad + rows0 + r) * width + c * 8);
  }
  float m_run[MT][2], l_run[MT][2], acc[MT][MAX_NTW][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
    for (int nt = 0; nt < MAX_NTW; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;
  }
  const int ntw = rank / 32;                         // n-tiles of L that this warp owns
  const int col0 = warp * (rank / 4);

  for (int tile = t_lo; tile < t_hi; ++tile) {
    __syncthreads();                                 // the tile before is no longer read (and qa_s is written)
    const int page = kv.page_table[(size_t)slot * kv.table_width + (tile % kv.ring_pages)];
    const bool page_ok = page >= 0 && page < kv.n_pages;
    if (!page_ok && tid == 0) atomicOr(err, IERT_ERR_PAGE_RANGE);
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(kv.k) + (size_t)(page_ok ? page : 0) * BK * width;
    const int valid = page_ok ? min(BK, n_keys - tile * BK) : 0;     // rows beyond hold other sequences' leftovers
    for (int i = tid; i < BK * chunks; i += THREADS) {
      const int r = i / chunks, c = i - r * chunks;
      __nv_bfloat16* dst = c_s + r * ldc + c * 8;
      if (r < valid)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src + (size_t)r * width + c * 8));
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // ---- scores of this warp's 16 keys for all heads of the CTA
    float sc[MT][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) sc[mt][nt][0] = sc[mt][nt][1] = sc[mt][nt][2] = sc[mt][nt][3] = 0.f;
    for (int k0 = 0; k0 < width; k0 += 16) {
      uint32_t bf[2][2];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const __nv_bfloat16* row = c_s + (warp * 16 + nt * 8 + g) * ldc + k0 + 2 * t4;
        bf[nt][0] = lds32(row);
        bf[nt][1] = lds32(row + 8);
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const __nv_bfloat16* row = qa_s + (mt * 16 + g) * ldc + k0 + 2 * t4;
        const uint32_t a[4] = {lds32(row), lds32(row + 8 * ldc), lds32(row + 8), lds32(row + 8 * ldc + 8)};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) mma_bf16(sc[mt][nt], a, bf[nt][0], bf[nt][1]);
      }
    }
    // ---- scale, mask, row maxima over the whole tile
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = warp * 16 + nt * 8 + 2 * t4 + e;
            const float v = j < valid ? sc[mt][nt][half * 2 + e] * scale : -INFINITY;
            sc[mt][nt][half * 2 + e] = v;
            mx = fmaxf(mx, v);
          }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        if (t4 == 0) wmax[warp * MT * 16 + mt * 16 + half * 8 + g] = mx;
      }
    __syncthreads();
    float alpha[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = mt * 16 + half * 8 + g;
        float m_new = m_run[mt][half];
#pragma unroll
        for (int w = 0; w < 4; ++w) m_new = fmaxf(m_new, wmax[w * MT * 16 + row]);
        alpha[mt][half] = m_run[mt][half] == -INFINITY ? 0.f : expf(m_run[mt][half] - m_new);
        m_run[mt][half] = m_new;                     // finite: every tile of a run holds at least one key
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const float p0 = sc[mt][nt][half * 2] == -INFINITY ? 0.f : expf(sc[mt][nt][half * 2] - m_new);
          const float p1 = sc[mt][nt][half * 2 + 1] == -INFINITY ? 0.f : expf(sc[mt][nt][half * 2 + 1] - m_new);
          sum += p0 + p1;
          *reinterpret_cast<__nv_bfloat162*>(p_s + row * PLD + warp * 16 + nt * 8 + 2 * t4) = __floats2bfloat162_rn(p0, p1);
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (t4 == 0) wsum[warp * MT * 16 + row] = sum;
      }
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = mt * 16 + half * 8 + g;
        l_run[mt][half] = l_run[mt][half] * alpha[mt][half] +
                          ((wsum[row] + wsum[MT * 16 + row]) + (wsum[2 * MT * 16 + row] + wsum[3 * MT * 16 + row]));
      }
    // ---- L += P C for this warp's rank columns
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < MAX_NTW; ++nt)
        if (nt < ntw) {
          acc[mt][nt][0] *= alpha[mt][0]; acc[mt][nt][1] *= alpha[mt][0];
          acc[mt][nt][2] *= alpha[mt][1]; acc[mt][nt][3] *= alpha[mt][1];
        }
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      uint32_t a[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const __nv_bfloat16* row = p_s + (mt * 16 + g) * PLD + ks * 16 + 2 * t4;
        a[mt][0] = lds32(row); a[mt][1] = lds32(row + 8 * PLD); a[mt][2] = lds32(row + 8); a[mt][3] = lds32(row + 8 * PLD + 8);
      }
      const __nv_bfloat16* krow = c_s + (ks * 16 + (lane & 15)) * ldc + col0;
#pragma unroll
      for (int nt = 0; nt < MAX_NTW; ++nt)
        if (nt < ntw) {
          uint32_t b0, b1;
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(smem_u32(krow + nt * 8)));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) mma_bf16(acc[mt][nt], a[mt], b0, b1);
        }
    }
  }
  // ---- this run's partial result
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const size_t row = part_row0 + mt * 16 + half * 8 + g;
      if (warp == 0 && t4 == 0) { part_m[row] = m_run[mt][half]; part_l[row] = l_run[mt][half]; }
#pragma unroll
      for (int nt = 0; nt < MAX_NTW; ++nt)
        if (nt < ntw)
          *reinterpret_cast<float2*>(part_acc + row * rank + col0 + nt * 8 + 2 * t4) =
              make_float2(acc[mt][nt][half * 2], acc[mt][nt][half * 2 + 1]);
    }
}

constexpr int MERGE_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(MERGE_THREADS)
latent_decode_merge_kernel(const float* __restrict__ part_m, const float* __restrict__ part_l,
                           const float* __restrict__ part_acc, int splits, int Hpad, int rank,
                           const float* __restrict__ sink, const float* __restrict__ gate, const T* __restrict__ w_uv,
                           T* __restrict__ out, IertBatchView b, int H, int V) {
  extern __shared__ float sm[];
  float* lat = sm;                 // [rank]
  float* wgt = sm + rank;          // [64]
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  T* o = out + ((size_t)t * H + h) * V;
  if (b.slot_ids[t] < 0) {
    for (int e = threadIdx.x; e < V; e += MERGE_THREADS) o[e] = from_f32<T>(0.f);
    return;
  }
  if (threadIdx.x < 32) {                 // splits <= 64: two runs per lane
    const int lane = threadIdx.x;
    float mi[2], li[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = lane + 32 * k;
      const size_t row = ((size_t)t * splits + (i < splits ? i : 0)) * Hpad + h;
      mi[k] = i < splits ? part_m[row] : -INFINITY;
      li[k] = i < splits ? part_l[row] : 0.f;
    }
    const float snk = sink ? sink[h] : -INFINITY;
    const float M = fmaxf(warp_max(fmaxf(mi[0], mi[1])), snk);
    float w[2], part = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      w[k] = mi[k] == -INFINITY ? 0.f : expf(mi[k] - M);
      part += w[k] * li[k];
    }
    const float L = warp_sum(part) + (sink ? expf(snk - M) : 0.f);
    const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) wgt[lane + 32 * k] = lane + 32 * k < splits ? w[k] * inv : 0.f;
  }
  __syncthreads();
  // the runs' partial sums, eight loads in flight per thread; an empty run's row (weight 0) is never read
  for (int r = threadIdx.x; r < rank; r += MERGE_THREADS) {
    float a = 0.f;
    for (int i0 = 0; i0 < splits; i0 += 8) {
      float v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int i = i0 + k;
        v[k] = (i < splits && wgt[i] != 0.f) ? part_acc[(((size_t)t * splits + i) * Hpad + h) * rank + r] : 0.f;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) a = fmaf(wgt[(i0 + k) & 63], v[k], a);
    }
    lat[r] = a;
  }
  __syncthreads();
  // W_uv: rank is a multiple of 32, 16-byte loads of eight weights; eight rows' loads are issued before the first is used
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e0 = warp * 8; e0 < V; e0 += (MERGE_THREADS / 32) * 8) {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = lane * 8; r < rank; r += 32 * 8) {
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        v[k] = e0 + k < V ? *reinterpret_cast<const uint4*>(w_uv + ((size_t)h * V + e0 + k) * rank + r) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float2 f = __bfloat1622float2(p[c]);
          a[k] = fmaf(f.x, lat[r + 2 * c], a[k]);
          a[k] = fmaf(f.y, lat[r + 2 * c + 1], a[k]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sum = warp_sum(a[k]);
      if (lane == 0 && e0 + k < V) o[e0 + k] = from_f32<T>(gate ? sum * gate[(size_t)t * H + h] : sum);
    }
  }
}

size_t decode_smem(int mt, int width) {
  return (size_t)(mt * 16 + BK) * (width + 8) * 2 + (size_t)mt * 16 * PLD * 2 + (size_t)8 * mt * 16 * 4;
}

}  // namespace

// Heads padded to whole MMA tiles (16, or 32 from 17 heads on), and how many runs of tiles a sequence is cut into.
IERT_API int iert_latent_decode_tc_plan(int n_seqs, int H, int table_width, int* Hpad, int* splits) {
  const int tiles = (H + 15) / 16, mt = tiles >= 2 ? 2 : 1;
  const int groups = (tiles + mt - 1) / mt;
  *Hpad = groups * mt * 16;
  int want = (2 * iert_sm_count_cached() + n_seqs * groups - 1) / (n_seqs * groups > 0 ? n_seqs * groups : 1);
  if (want > 32) want = 32;
  // a run's partial result (heads x rank floats) is as many bytes as 16 or more cached rows: runs of fewer than
  // four tiles of the longest sequence the cache can hold cost more than they spread
  if (want > (table_width + 3) / 4) want = (table_width + 3) / 4;
  if (want < 1) want = 1;
  *splits = want;
  return IERT_OK;
}

// q [T, ldq] bf16 (H*(D+R) per token, one token per sequence: per head D unrotated and R rotated numbers); the cache's
// rows are rank + R wide (latent | rotated key part); w_uk [H*D, rank], w_uv [H*V, rank] bf16 row-major; gate: fp32 [T, H]
// or null.  qa: scratch bf16 [T, Hpad, rank + R]; part_m, part_l: fp32 [T, splits, Hpad]; part_acc: fp32 [T, splits, Hpad, rank];
// out bf16 [T, H*V].  Hpad and splits as iert_latent_decode_tc_plan gives them.
IERT_API int iert_latent_attention_decode_tc(const void* q, long long ldq, const void* w_uk, const void* w_uv, void* out,
                                             const IertBatchView* batch, const IertKvView* kv, int H, int D, int R, int V,
                                             float scale, const float* sink, const float* gate, int Hpad, int splits,
                                             void* qa, float* part_m, float* part_l, float* part_acc, int* err,
                                             cudaStream_t stream) {
  const int T = batch->n_tokens, width = kv->head_dim, rank = width - R;
  if (T <= 0) return IERT_OK;
  if (T != batch->n_seqs || kv->dtype != IERT_BF16 || kv->kv_heads != 1 || kv->page_tokens != BK || rank % 32 || R < 0 ||
      R % 16 || width > 640 || rank < 32 || rank > MAX_NTW * 32 || H <= 0 || Hpad % 16 || Hpad < H || Hpad > 65535 || splits < 1 || splits > 64 ||
      D <= 0 || D > 8192 || V <= 0 || (ldq % 8) || ((uintptr_t)q & 15))
    return IERT_BAD_ARGUMENT;
  const int mt = Hpad % 32 == 0 ? 2 : 1;
  const size_t smem = decode_smem(mt, width);
  static bool configured = false;
  if (!configured) {
    const int most = (int)decode_smem(2, 640);
    if (cudaFuncSetAttribute(latent_decode_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess ||
        cudaFuncSetAttribute(latent_decode_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess) {
      cudaGetLastError();
      return IERT_CUDA_ERROR;
    }
    configured = true;
  }
  launch_dep(latent_absorb_q_kernel, dim3(T, Hpad), dim3(ABSORB_THREADS), (size_t)(D + 4 * rank) * sizeof(float), stream,
             (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)w_uk, (__nv_bfloat16*)qa, H, Hpad, D, R, rank);
  dim3 grid(T, splits, Hpad / (mt * 16));
  if (mt == 2)
    launch_dep(latent_decode_tc_kernel<2>, grid, dim3(THREADS), smem, stream, (const __nv_bfloat16*)qa, *batch, *kv, Hpad, R,
               scale, splits, part_m, part_l, part_acc, err);
  else
    launch_dep(latent_decode_tc_kernel<1>, grid, dim3(THREADS), smem, stream, (const __nv_bfloat16*)qa, *batch, *kv, Hpad, R,
               scale, splits, part_m, part_l, part_acc, err);
  launch_dep(latent_decode_merge_kernel<__nv_bfloat16>, dim3(T, H), dim3(MERGE_THREADS), (size_t)(rank + 64) * sizeof(float),
             stream, (const float*)part_m, (const float*)part_l, (const float*)part_acc, splits, Hpad, rank, sink, gate,
             (const __nv_bfloat16*)w_uv, (__nv_bfloat16*)out, *batch, H, V);
  return iert_check_launch("latent_attention_decode_tc");
}
