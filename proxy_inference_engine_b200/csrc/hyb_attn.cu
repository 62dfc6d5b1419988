// Differential attention over 64-token pages, ragged steps.  A query head carries TWO maps (two query / key vectors of d
// features) over the same values:  o = unit_rms(softmax(s1) V - lambda softmax(s2) V) * out_scale,
// s = softcap * tanh(q . k * scale / softcap), keys visible inside a sliding window that ends at the query's own position.
// attn_prepare_kernel  per token: RMS norm of every (head, map) of q and k with a shared plain weight, rotation of adjacent
//                      feature pairs of the first rot_dims features (angle = position x frequency, evaluated in double),
//                      k and v written to the sequence's page at the token's position
// attn_run_kernel      one CTA per (token, query head): 4 warps take 32-key blocks of the window in turn, a lane scores
//                      one key for both maps, the warp keeps an online softmax per map and accumulates p V with the lanes
//                      spread over the value features; the warps merge through shared memory
// A step's keys are appended before its queries run, so a prompt portion sees itself through the same pages as its past.
#include "hyb_common.cuh"

namespace pieh {

constexpr int kPage = 64;

template <typename KT>
__global__ void __launch_bounds__(128) attn_prepare_kernel(float* q_out, const float* proj, long long ld, const pieh_attn a,
                                                           const pieh_batch b) {
  extern __shared__ float cs[];   // [rot_dims / 2][2]: cos, sin of this token's angles
  const int t = blockIdx.x;
  const int i = b.tok_seq[t], p = b.tok_pos[t];
  for (int f = threadIdx.x; f < a.rot_dims / 2; f += blockDim.x) {
    double s, c;
    sincos((double)p * a.rot_freqs[f], &s, &c);
    cs[2 * f] = (float)c;
    cs[2 * f + 1] = (float)s;
  }
  __syncthreads();
  const size_t slot = (size_t)b.block_table[(size_t)i * b.bt_stride + p / kPage] * kPage + p % kPage;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int d = a.d, nqu = a.H * 2, nku = a.G * 2;
  const float* row = proj + (size_t)t * ld;
  KT* kp = reinterpret_cast<KT*>(a.k_pages) + slot * nku * d;
  for (int u = warp; u < nqu + nku; u += nw) {   // units: (head, map) of q, then of k
    const float* src = row + (size_t)u * d;
    const float* wn = u < nqu ? a.q_norm : a.k_norm;
    float inv = 1.f;
    if (wn) {
      float ss = 0.f;
      for (int c = lane; c < d; c += 32) ss = fmaf(src[c], src[c], ss);
      ss = warp_sum(ss);
      inv = 1.f / sqrtf(ss / (float)d + a.eps);
    }
    for (int pi = lane; 2 * pi < d; pi += 32) {
      const int e0 = 2 * pi, e1 = e0 + 1;
      float x0 = src[e0] * inv * (wn ? wn[e0] : 1.f);
      float x1 = e1 < d ? src[e1] * inv * (wn ? wn[e1] : 1.f) : 0.f;
      if (e1 < a.rot_dims) {
        const float c = cs[2 * pi], s = cs[2 * pi + 1];
        const float y0 = x0 * c - x1 * s, y1 = x1 * c + x0 * s;
        x0 = y0; x1 = y1;
      }
      if (u < nqu) {
        float* dst = q_out + ((size_t)t * nqu + u) * d;
        dst[e0] = x0;
        if (e1 < d) dst[e1] = x1;
      } else {
        KT* dst = kp + (size_t)(u - nqu) * d;
        elem<KT>::store(dst + e0, x0);
        if (e1 < d) elem<KT>::store(dst + e1, x1);
      }
    }
  }
  KT* vp = reinterpret_cast<KT*>(a.v_pages) + slot * a.G * a.dv;
  const float* vsrc = row + (size_t)(nqu + nku) * d;
  for (int c = threadIdx.x; c < a.G * a.dv; c += blockDim.x) elem<KT>::store(vp + c, vsrc[c]);
}

template <typename KT, typename OT, int NV>
__global__ void __launch_bounds__(128) attn_run_kernel(OT* out, const float* q, const pieh_attn a, const pieh_batch b) {
  extern __shared__ float sm[];
  __shared__ float red[33];
  const int t = blockIdx.x / a.H, h = blockIdx.x - t * a.H;
  const int g = h / (a.H / a.G);
  const int i = b.tok_seq[t], p = b.tok_pos[t];
  const int d = a.d, dv = a.dv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = sm;                  // [2][d]
  float* mg = qs + 2 * d;          // [4 warps][2 maps][dv + 2]: acc, m, l
  for (int c = threadIdx.x; c < 2 * d; c += 128) qs[c] = q[((size_t)t * a.H + h) * 2 * d + c];
  __syncthreads();
  const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
  const int32_t* table = b.block_table + (size_t)i * b.bt_stride;
  const KT* kpool = reinterpret_cast<const KT*>(a.k_pages);
  const KT* vpool = reinterpret_cast<const KT*>(a.v_pages);
  float m1 = -1e30f, m2 = -1e30f, l1 = 0.f, l2 = 0.f, acc1[NV], acc2[NV];
#pragma unroll
  for (int x = 0; x < NV; ++x) acc1[x] = acc2[x] = 0.f;
  for (int base = lo + warp * 32; base <= p; base += 128) {
    const int j = base + lane;
    const bool ok = j <= p;
    long long slot = 0;
    float s1 = -1e30f, s2 = -1e30f;
    if (ok) {
      slot = (long long)table[j / kPage] * kPage + j % kPage;
      const KT* kr = kpool + ((size_t)slot * a.G + g) * 2 * d;
      float d1 = 0.f, d2 = 0.f;
      for (int c = 0; c < d; ++c) {
        d1 = fmaf(qs[c], elem<KT>::load(kr + c), d1);
        d2 = fmaf(qs[d + c], elem<KT>::load(kr + d + c), d2);
      }
      s1 = d1 * a.scale; s2 = d2 * a.scale;
      if (a.softcap > 0.f) { s1 = a.softcap * tanhf(s1 / a.softcap); s2 = a.softcap * tanhf(s2 / a.softcap); }
    }
    const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
    const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);
    const float p1 = ok ? expf(s1 - n1) : 0.f, p2 = ok ? expf(s2 - n2) : 0.f;
    l1 = l1 * c1 + warp_sum(p1);
    l2 = l2 * c2 + warp_sum(p2);
    m1 = n1; m2 = n2;
#pragma unroll
    for (int x = 0; x < NV; ++x) { acc1[x] *= c1; acc2[x] *= c2; }
    const int cnt = min(32, p - base + 1);
    for (int kk = 0; kk < cnt; ++kk) {
      const float w1 = __shfl_sync(0xffffffffu, p1, kk), w2 = __shfl_sync(0xffffffffu, p2, kk);
      const long long sl = __shfl_sync(0xffffffffu, slot, kk);
      const KT* vr = vpool + ((size_t)sl * a.G + g) * dv;
#pragma unroll
      for (int x = 0; x < NV; ++x) {
        const int c = lane + 32 * x;
        if (c < dv) {
          const float vv = elem<KT>::load(vr + c);
          acc1[x] = fmaf(w1, vv, acc1[x]);
          acc2[x] = fmaf(w2, vv, acc2[x]);
        }
      }
    }
  }
  float* mine = mg + (size_t)warp * 2 * (dv + 2);
#pragma unroll
  for (int x = 0; x < NV; ++x) {
    const int c = lane + 32 * x;
    if (c < dv) { mine[c] = acc1[x]; mine[dv + 2 + c] = acc2[x]; }
  }
  if (lane == 0) { mine[dv] = m1; mine[dv + 1] = l1; mine[2 * dv + 2] = m2; mine[2 * dv + 3] = l2; }
  __syncthreads();
  float ssq = 0.f;
  float ov[(NV + 3) / 4];   // features this thread owns: c = threadIdx.x + 128 * y
#pragma unroll
  for (int y = 0; y < (NV + 3) / 4; ++y) {
    const int c = threadIdx.x + 128 * y;
    ov[y] = 0.f;
    if (c < dv) {
      float res[2];
      for (int mp = 0; mp < 2; ++mp) {
        float M = -1e30f;
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mg[(size_t)(w * 2 + mp) * (dv + 2) + dv]);
        float L = 0.f, A = 0.f;
        for (int w = 0; w < 4; ++w) {
          const float* src = mg + (size_t)(w * 2 + mp) * (dv + 2);
          const float f = expf(src[dv] - M);
          L = fmaf(src[dv + 1], f, L);
          A = fmaf(src[c], f, A);
        }
        res[mp] = A / L;
      }
      ov[y] = res[0] - a.lambda * res[1];
      ssq = fmaf(ov[y], ov[y], ssq);
    }
  }
  ssq = block_sum(ssq, red);
  const float inv = a.out_scale / sqrtf(ssq / (float)dv + a.eps);
#pragma unroll
  for (int y = 0; y < (NV + 3) / 4; ++y) {
    const int c = threadIdx.x + 128 * y;
    if (c < dv) elem<OT>::store(out + ((size_t)t * a.H + h) * dv + c, ov[y] * inv);
  }
}

static bool attn_ok(const pieh_attn* a) {
  return a && a->H > 0 && a->G > 0 && a->H % a->G == 0 && a->d > 0 && a->dv > 0 && a->dv <= 256 && a->d <= 1024 &&
         a->rot_dims >= 0 && a->rot_dims <= a->d && a->rot_dims % 2 == 0 && (a->rot_dims == 0 || a->rot_freqs) &&
         a->k_pages && a->v_pages && ((a->q_norm == nullptr) == (a->k_norm == nullptr));
}

template <typename KT, typename OT>
static cudaError_t launch_run(OT* out, const float* q, const pieh_attn& a, const pieh_batch& b, cudaStream_t st) {
  const size_t smem = ((size_t)2 * a.d + 8 * (a.dv + 2)) * 4;
  const unsigned grid = (unsigned)b.T * a.H;
  const int nv = (a.dv + 31) / 32;
  if (nv <= 1) attn_run_kernel<KT, OT, 1><<<grid, 128, smem, st>>>(out, q, a, b);
  else if (nv <= 2) attn_run_kernel<KT, OT, 2><<<grid, 128, smem, st>>>(out, q, a, b);
  else if (nv <= 4) attn_run_kernel<KT, OT, 4><<<grid, 128, smem, st>>>(out, q, a, b);
  else attn_run_kernel<KT, OT, 8><<<grid, 128, smem, st>>>(out, q, a, b);
  return cudaGetLastError();
}

}  // namespace pieh

using namespace pieh;

extern "C" int pieh_attn_prepare(float* q_out, const float* proj, long long ld, const pieh_attn* a, const pieh_batch* b,
                                 void* stream) {
  if (!q_out || !proj || !a || !b) return PIE_ENULL;
  if (!attn_ok(a)) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  const size_t smem = (size_t)(a->rot_dims + 2) * 4;
  count_launch();
  PIEH_DISPATCH_DTYPE(a->kv_dtype, KT, (attn_prepare_kernel<KT><<<b->T, 128, smem, (cudaStream_t)stream>>>(q_out, proj, ld, *a, *b)));
  return status_of(cudaGetLastError());
}

extern "C" int pieh_attn_run(void* out, int out_dtype, const float* q, const pieh_attn* a, const pieh_batch* b,
                             void* stream) {
  if (!out || !q || !a || !b) return PIE_ENULL;
  if (!attn_ok(a)) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  typedef __nv_bfloat16 bf;
  count_launch();
  cudaError_t e;
  if (a->kv_dtype == PIE_DTYPE_BF16)
    e = out_dtype == PIE_DTYPE_BF16 ? launch_run<bf, bf>((bf*)out, q, *a, *b, st) : launch_run<bf, float>((float*)out, q, *a, *b, st);
  else
    e = out_dtype == PIE_DTYPE_BF16 ? launch_run<float, bf>((bf*)out, q, *a, *b, st) : launch_run<float, float>((float*)out, q, *a, *b, st);
  return status_of(e);
}
