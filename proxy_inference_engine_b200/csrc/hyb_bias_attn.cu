// Attention with a per-head linear distance bias, a softmax sink and a sigmoid output gate over 64-token pages, ragged steps.
//   s_ij = q_i . k_j * scale - slope_h (i - j),  j <= i (and i - j < window if one is set)
//   p_ij = exp(s_ij) / (sink + sum_j exp(s_ij))          sink = 1: a term of score 0 that carries no value, so a query
//                                                        that matches nothing returns (almost) nothing
//   out_i = sum_j p_ij v_j * sigmoid(gate_i)
// bias_prepare_kernel   per token: ONE rms norm over all heads' query features (and one over all key features) with
//                       per-feature weights, the query temperature 1 + c ln(floor((p + 1) / every) + 1), then the normed
//                       keys go to the key pages and the values -- here usually the PROJECTED keys themselves, v_off ==
//                       k_off -- to the value pages at the token's position
// bias_run_kernel       one CTA per (token, query head): 8 warps take 32-key blocks in turn with an online softmax each,
//                       merged through shared memory together with the sink; serves decoding and every fp32 step
// bias_tile_kernel      prompt portions over bf16 pages: 64-row query tiles on mma.sync (below)
// A step's keys are appended before its queries run, so a prompt portion sees itself through the same pages as its past.
#include "hyb_common.cuh"

namespace pieh {

constexpr int kPage = 64;

template <typename KT>
__global__ void __launch_bounds__(256) bias_prepare_kernel(float* q_out, const float* proj, long long ld,
                                                           const pieh_bias_attn a, const pieh_batch b) {
  __shared__ float red[33];
  pdl_sync();
  const int t = blockIdx.x;
  const int i = b.tok_seq[t], p = b.tok_pos[t];
  const int nq = a.H * a.d, nk = a.G * a.d, nv = a.G * a.dv;
  const float* row = proj + (size_t)t * ld;
  float iq = 1.f, ik = 1.f;
  if (a.q_norm) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
    iq = 1.f / sqrtf(block_sum(ss, red) / (float)nq + a.eps);
  }
  if (a.k_norm) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < nk; c += blockDim.x) ss = fmaf(row[a.k_off + c], row[a.k_off + c], ss);
    ik = 1.f / sqrtf(block_sum(ss, red) / (float)nk + a.eps);
  }
  if (a.temp_every > 0) iq *= 1.f + a.temp_coef * logf((float)((p + 1) / a.temp_every) + 1.f);
  const size_t slot = (size_t)b.block_table[(size_t)i * b.bt_stride + p / kPage] * kPage + p % kPage;
  KT* kp = reinterpret_cast<KT*>(a.k_pages) + slot * nk;
  KT* vp = reinterpret_cast<KT*>(a.v_pages) + slot * nv;
  for (int c = threadIdx.x; c < nq; c += blockDim.x) q_out[(size_t)t * nq + c] = row[c] * iq * (a.q_norm ? a.q_norm[c] : 1.f);
  for (int c = threadIdx.x; c < nk; c += blockDim.x)
    elem<KT>::store(kp + c, row[a.k_off + c] * ik * (a.k_norm ? a.k_norm[c] : 1.f));
  for (int c = threadIdx.x; c < nv; c += blockDim.x) elem<KT>::store(vp + c, row[a.v_off + c]);
}

constexpr int kRunWarps = 8;

template <typename T> struct ld8;   // 8 consecutive cache elements as floats
template <> struct ld8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct ld8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
};

template <typename KT, typename OT, int NV>
__global__ void __launch_bounds__(kRunWarps * 32) bias_run_kernel(OT* out, const float* q, const float* proj, long long ld,
                                                                  const pieh_bias_attn a, const pieh_batch b) {
  extern __shared__ __align__(16) float sm[];
  constexpr int NW = kRunWarps, NTH = kRunWarps * 32;
  pdl_sync();
  const int t = blockIdx.x / a.H, h = blockIdx.x - t * a.H;
  const int g = h / (a.H / a.G);
  const int i = b.tok_seq[t], p = b.tok_pos[t];
  const int d = a.d, dv = a.dv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = sm;              // [d]
  float* mg = qs + d;          // [warps][dv + 2]: acc, m, l
  for (int c = threadIdx.x; c < d; c += NTH) qs[c] = q[((size_t)t * a.H + h) * d + c];
  __syncthreads();
  const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
  const float slope = a.slopes ? a.slopes[h] : 0.f;
  const int32_t* table = b.block_table + (size_t)i * b.bt_stride;
  const KT* kpool = reinterpret_cast<const KT*>(a.k_pages);
  const KT* vpool = reinterpret_cast<const KT*>(a.v_pages);
  const bool vec = (d & 7) == 0;
  float m = -1e30f, l = 0.f, acc[NV];
#pragma unroll
  for (int x = 0; x < NV; ++x) acc[x] = 0.f;
  for (int base = lo + warp * 32; base <= p; base += NW * 32) {
    const int j = base + lane;
    const bool ok = j <= p;
    long long slot = 0;
    float s = -1e30f;
    if (ok) {
      slot = (long long)table[j / kPage] * kPage + j % kPage;
      const KT* kr = kpool + ((size_t)slot * a.G + g) * d;
      float dot = 0.f;
      if (vec) {
#pragma unroll 4
        for (int c = 0; c < d; c += 8) {
          float kk[8];
          ld8<KT>::load(kr + c, kk);
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(qs[c + e], kk[e], dot);
        }
      } else {
        for (int c = 0; c < d; ++c) dot = fmaf(qs[c], elem<KT>::load(kr + c), dot);
      }
      s = dot * a.scale - slope * (float)(p - j);
    }
    const float n = fmaxf(m, warp_max(s));
    const float cf = expf(m - n);
    const float pj = ok ? expf(s - n) : 0.f;
    l = l * cf + warp_sum(pj);
    m = n;
#pragma unroll
    for (int x = 0; x < NV; ++x) acc[x] *= cf;
#pragma unroll 1
    for (int k0 = 0; k0 < 32; k0 += 4) {
      if (base + k0 > p) break;
      float w[4], vv[4][NV];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        w[u] = __shfl_sync(0xffffffffu, pj, k0 + u);
        const long long sl = __shfl_sync(0xffffffffu, slot, k0 + u);
        const KT* vr = vpool + ((size_t)sl * a.G + g) * dv;
#pragma unroll
        for (int x = 0; x < NV; ++x) {
          const int c = lane + 32 * x;
          vv[u][x] = c < dv ? elem<KT>::load(vr + c) : 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int x = 0; x < NV; ++x) acc[x] = fmaf(w[u], vv[u][x], acc[x]);
    }
  }
  float* mine = mg + (size_t)warp * (dv + 2);
#pragma unroll
  for (int x = 0; x < NV; ++x) {
    const int c = lane + 32 * x;
    if (c < dv) mine[c] = acc[x];
  }
  if (lane == 0) { mine[dv] = m; mine[dv + 1] = l; }
  __syncthreads();
  const int c = threadIdx.x;   // dv <= 256 = threads
  if (c < dv) {
    float M = a.sink ? 0.f : -1e30f;   // the sink is one more partial softmax: maximum 0, sum 1, no values
    for (int w = 0; w < NW; ++w) M = fmaxf(M, mg[(size_t)w * (dv + 2) + dv]);
    float L = a.sink ? expf(-M) : 0.f, A = 0.f;
    for (int w = 0; w < NW; ++w) {
      const float* src = mg + (size_t)w * (dv + 2);
      const float f = expf(src[dv] - M);
      L = fmaf(src[dv + 1], f, L);
      A = fmaf(src[c], f, A);
    }
    float o = A / L;
    if (a.g_off >= 0) o *= 1.f / (1.f + expf(-proj[(size_t)t * ld + a.g_off + (size_t)h * dv + c]));
    elem<OT>::store(out + ((size_t)t * a.H + h) * dv + c, o);
  }
}

static bool bias_attn_ok(const pieh_bias_attn* a) {
  return a && a->H > 0 && a->G > 0 && a->H % a->G == 0 && a->d > 0 && a->dv > 0 && a->dv <= 256 && a->d <= 1024 &&
         a->k_pages && a->v_pages && a->temp_every >= 0 && a->window >= 0 && a->k_off >= 0 && a->v_off >= 0;
}

template <typename KT, typename OT>
static cudaError_t launch_run(OT* out, const float* q, const float* proj, long long ld, const pieh_bias_attn& a,
                              const pieh_batch& b, cudaStream_t st) {
  const size_t smem = ((size_t)a.d + kRunWarps * (a.dv + 2)) * 4;
  const unsigned grid = (unsigned)b.T * a.H;
  const int nv = (a.dv + 31) / 32, nth = kRunWarps * 32;
  if (nv <= 1) return launch_k(bias_run_kernel<KT, OT, 1>, dim3(grid), dim3(nth), smem, st, out, q, proj, ld, a, b);
  if (nv <= 2) return launch_k(bias_run_kernel<KT, OT, 2>, dim3(grid), dim3(nth), smem, st, out, q, proj, ld, a, b);
  if (nv <= 4) return launch_k(bias_run_kernel<KT, OT, 4>, dim3(grid), dim3(nth), smem, st, out, q, proj, ld, a, b);
  return launch_k(bias_run_kernel<KT, OT, 8>, dim3(grid), dim3(nth), smem, st, out, q, proj, ld, a, b);
}

}  // namespace pieh

using namespace pieh;

extern "C" int pieh_bias_attn_prepare(float* q_out, const float* proj, long long ld, const pieh_bias_attn* a,
                                      const pieh_batch* b, void* stream) {
  if (!q_out || !proj || !a || !b) return PIE_ENULL;
  if (!bias_attn_ok(a)) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  count_launch();
  PIEH_DISPATCH_DTYPE(a->kv_dtype, KT, launch_k(bias_prepare_kernel<KT>, dim3(b->T), dim3(256), 0, (cudaStream_t)stream, q_out, proj, ld, *a, *b));
  return status_of(cudaGetLastError());
}

extern "C" int pieh_bias_attn_run(void* out, int out_dtype, const float* q, const float* proj, long long ld,
                                  const pieh_bias_attn* a, const pieh_batch* b, void* stream) {
  if (!out || !q || !a || !b || (a->g_off >= 0 && !proj)) return PIE_ENULL;
  if (!bias_attn_ok(a)) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  typedef __nv_bfloat16 bf;
  count_launch();
  cudaError_t e;
  if (a->kv_dtype == PIE_DTYPE_BF16)
    e = out_dtype == PIE_DTYPE_BF16 ? launch_run<bf, bf>((bf*)out, q, proj, ld, *a, *b, st)
                                    : launch_run<bf, float>((float*)out, q, proj, ld, *a, *b, st);
  else
    e = out_dtype == PIE_DTYPE_BF16 ? launch_run<float, bf>((bf*)out, q, proj, ld, *a, *b, st)
                                    : launch_run<float, float>((float*)out, q, proj, ld, *a, *b, st);
  return status_of(e);
}
