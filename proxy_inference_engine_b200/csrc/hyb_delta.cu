// Gated delta rule over ragged steps: a matrix state S [dk, dv] per (sequence, head) in fp32, carried in a slot.
//   per token:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// delta_prepare_kernel  short causal convolution (history of taps - 1 inputs per sequence slot) + silu on q, k, v; q and k
//                       to unit length (q also times dk^-1/2); beta = sigmoid(.), g = exp(-exp(A_log) softplus(. + dt_bias))
// conv_advance_kernel   moves every sequence's convolution history past this step's rows
// delta_scan_kernel     the recurrence: a column of S lives in the registers of R adjacent lanes (RPT rows each), so a
//                       token costs 3 RPT multiply-adds and two log2(R)-step shuffles per thread and no barrier; the
//                       step's q / k / v rows are staged through shared memory a chunk of tokens at a time
// delta_gate_kernel     per-head RMS norm of o, times the norm weight, times silu(gate)
// Everything that enters the recurrence is fp32; only delta_gate's output takes the act dtype.
#include "hyb_common.cuh"

namespace pieh {

constexpr int kMaxTaps = 8;

// grid (T, 2 G + H): one CTA per token and head-sized unit -- the G heads of q, the G heads of k, the H heads of v
__global__ void __launch_bounds__(128) delta_prepare_kernel(float* q, float* k, float* v, float* beta, float* decay,
                                                            const float* proj, long long ld, const pieh_delta d,
                                                            const pieh_batch b) {
  __shared__ float red[33];
  pdl_sync();
  const int t = blockIdx.x, u = blockIdx.y;
  const int i = b.tok_seq[t], start = b.seq_start[i], ctx = b.seq_ctx[i], slot = b.seq_slot[i];
  const int j = t - start;
  const int nq = d.G * d.dk, C = 2 * nq + d.H * d.dv, taps = d.taps;
  const float* hist = d.conv_state + (size_t)slot * (taps - 1) * C;
  const bool is_v = u >= 2 * d.G;
  const int n = is_v ? d.dv : d.dk;
  const int base = is_v ? 2 * nq + (u - 2 * d.G) * d.dv : u * d.dk;
  float y[4], ss = 0.f;   // n <= 512
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int c = base + threadIdx.x + 128 * e;
    y[e] = 0.f;
    if (threadIdx.x + 128 * e < n) {
      float acc = 0.f;
      for (int r = 0; r < taps; ++r) {
        float x;
        if (r <= j) x = proj[(size_t)(t - r) * ld + c];
        else {
          const int back = r - j;   // 1 .. taps - 1 tokens before this step
          x = ctx - back >= 0 ? hist[(size_t)(taps - 1 - back) * C + c] : 0.f;
        }
        acc = fmaf(d.conv_w[(size_t)c * taps + (taps - 1 - r)], x, acc);
      }
      y[e] = silu_f(acc);
      ss = fmaf(y[e], y[e], ss);
    }
  }
  float inv = 1.f;
  float* dst;
  if (is_v) dst = v + (size_t)t * d.H * d.dv + (base - 2 * nq);
  else {
    ss = block_sum(ss, red);
    inv = 1.f / sqrtf(ss + 1e-6f);
    if (u < d.G) { inv *= 1.f / sqrtf((float)d.dk); dst = q + (size_t)t * nq + base; }
    else dst = k + (size_t)t * nq + (base - nq);
  }
#pragma unroll
  for (int e = 0; e < 4; ++e)
    if (threadIdx.x + 128 * e < n) dst[threadIdx.x + 128 * e] = y[e] * inv;
  if (u == 0) {
    const float* row = proj + (size_t)t * ld + C + d.H * d.dv;   // behind the gate columns: b, then a
    for (int h = threadIdx.x; h < d.H; h += 128) {
      beta[(size_t)t * d.H + h] = 1.f / (1.f + expf(-row[h]));
      decay[(size_t)t * d.H + h] = expf(-expf(d.A_log[h]) * softplus_f(row[d.H + h] + d.dt_bias[h]));
    }
  }
}

__global__ void conv_advance_kernel(const float* proj, long long ld, const pieh_delta d, const pieh_batch b) {
  pdl_sync();
  const int i = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int C = 2 * d.G * d.dk + d.H * d.dv, taps = d.taps;
  if (c >= C) return;
  const int start = b.seq_start[i], n = b.seq_len[i], ctx = b.seq_ctx[i];
  float* hist = d.conv_state + (size_t)b.seq_slot[i] * (taps - 1) * C;
  float nv[kMaxTaps];
  for (int jj = 0; jj < taps - 1; ++jj) {
    const int p = ctx + n - (taps - 1) + jj;   // position this entry has to hold afterwards
    float x = 0.f;
    if (p >= ctx) x = proj[(size_t)(start + p - ctx) * ld + c];
    else if (p >= 0) x = hist[(size_t)(p - ctx + taps - 1) * C + c];
    nv[jj] = x;
  }
  for (int jj = 0; jj < taps - 1; ++jj) hist[(size_t)jj * C + c] = nv[jj];
}

constexpr int kScanThreads = 128, kScanChunk = 16;

__device__ __forceinline__ void cp_async_f(float* smem_dst, const float* gsrc, int bytes) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gsrc) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gsrc) : "memory");
}

template <int RPT>
__global__ void __launch_bounds__(kScanThreads) delta_scan_kernel(float* o, const float* q, const float* k, const float* v,
                                                                  const float* beta, const float* decay,
                                                                  const pieh_delta d, const pieh_batch b, int R) {
  extern __shared__ __align__(16) float sm[];
  pdl_sync();
  const int cols = kScanThreads / R;
  const int h = blockIdx.y, i = blockIdx.z;
  const int hk = h / (d.H / d.G);
  const int start = b.seq_start[i], n = b.seq_len[i], ctx = b.seq_ctx[i];
  const int rl = threadIdx.x % R, cl = threadIdx.x / R;
  const int j = blockIdx.x * cols + cl;           // column of S (feature of v)
  const bool col_ok = j < d.dv;
  const int dk = d.dk, dv = d.dv;
  // two chunk buffers: while the recurrence walks one chunk of tokens, cp.async fills the other
  const int buf_floats = kScanChunk * (2 * dk + cols + 2);
  float* S_g = d.state + (((size_t)b.seq_slot[i] * d.H + h) * dk) * dv;
  float S[RPT];
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int row = r * R + rl;   // rows are dealt round-robin to the R lanes: lane rl reads bank-adjacent k, q entries
    S[r] = (ctx > 0 && col_ok && row < dk) ? S_g[(size_t)row * dv + j] : 0.f;
  }
  const bool vec = (dk & 3) == 0;
  auto fill = [&](int which, int c0) {
    float* ks = sm + which * buf_floats;
    float* qs = ks + kScanChunk * dk;
    float* vs = qs + kScanChunk * dk;
    float* gb = vs + kScanChunk * cols;
    const int nc = min(kScanChunk, n - c0);
    if (vec) {
      const int per = dk >> 2;
      for (int e = threadIdx.x; e < nc * per; e += kScanThreads) {
        const int tt = e / per, r = (e - tt * per) << 2;
        const size_t src = ((size_t)(start + c0 + tt) * d.G + hk) * dk + r;
        cp_async_f(ks + tt * dk + r, k + src, 16);
        cp_async_f(qs + tt * dk + r, q + src, 16);
      }
    } else {
      for (int e = threadIdx.x; e < nc * dk; e += kScanThreads) {
        const int tt = e / dk, r = e - tt * dk;
        const size_t src = ((size_t)(start + c0 + tt) * d.G + hk) * dk + r;
        cp_async_f(ks + e, k + src, 4);
        cp_async_f(qs + e, q + src, 4);
      }
    }
    for (int e = threadIdx.x; e < nc * cols; e += kScanThreads) {
      const int tt = e / cols, c = e - tt * cols;
      const int jj = min(blockIdx.x * cols + c, dv - 1);
      cp_async_f(vs + e, v + ((size_t)(start + c0 + tt) * d.H + h) * dv + jj, 4);
    }
    for (int e = threadIdx.x; e < nc; e += kScanThreads) {
      cp_async_f(gb + 2 * e, decay + (size_t)(start + c0 + e) * d.H + h, 4);
      cp_async_f(gb + 2 * e + 1, beta + (size_t)(start + c0 + e) * d.H + h, 4);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float out_prev = 0.f;   // this lane's share of the last token's read-out, not yet summed over the R lanes
  int row_prev = -1;
  fill(0, 0);
  for (int c0 = 0, which = 0; c0 < n; c0 += kScanChunk, which ^= 1) {
    const int nc = min(kScanChunk, n - c0);
    if (c0 + kScanChunk < n) {
      fill(which ^ 1, c0 + kScanChunk);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* ks = sm + which * buf_floats;
    const float* qs = ks + kScanChunk * dk;
    const float* vs = qs + kScanChunk * dk;
    const float* gb = vs + kScanChunk * cols;
    for (int tt = 0; tt < nc; ++tt) {
      const float g = gb[2 * tt], be = gb[2 * tt + 1];
      const float* kr = ks + tt * dk + rl;
      const float* qr = qs + tt * dk + rl;
      float kk[RPT], pp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        kk[r] = r * R + rl < dk ? kr[r * R] : 0.f;
        S[r] *= g;
        pp[r & 3] = fmaf(S[r], kk[r], pp[r & 3]);
      }
      float pred = (pp[0] + pp[1]) + (pp[2] + pp[3]);
      // the read-out of the PREVIOUS token is reduced over the R lanes together with this token's prediction: two
      // independent shuffle chains instead of two in a row on the recurrence's critical path
      for (int off = 1; off < R; off <<= 1) {
        pred += __shfl_xor_sync(0xffffffffu, pred, off);
        out_prev += __shfl_xor_sync(0xffffffffu, out_prev, off);
      }
      if (row_prev >= 0 && rl == 0 && col_ok) o[((size_t)row_prev * d.H + h) * dv + j] = out_prev;
      const float u = be * (vs[tt * cols + cl] - pred);
      float oo[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        S[r] = fmaf(kk[r], u, S[r]);
        oo[r & 3] = fmaf(S[r], r * R + rl < dk ? qr[r * R] : 0.f, oo[r & 3]);
      }
      out_prev = (oo[0] + oo[1]) + (oo[2] + oo[3]);
      row_prev = start + c0 + tt;
    }
    __syncthreads();   // everyone is done with this buffer before the next fill overwrites it
  }
  for (int off = 1; off < R; off <<= 1) out_prev += __shfl_xor_sync(0xffffffffu, out_prev, off);
  if (row_prev >= 0 && rl == 0 && col_ok) o[((size_t)row_prev * d.H + h) * dv + j] = out_prev;
  if (col_ok) {
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int row = r * R + rl;
      if (row < dk) S_g[(size_t)row * dv + j] = S[r];
    }
  }
}

template <typename OT>
__global__ void delta_gate_kernel(OT* out, const float* o, const float* proj, long long ld, long long gate_off,
                                  const pieh_delta d, int T) {
  pdl_sync();
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= T * d.H) return;
  const int t = w / d.H, h = w - t * d.H;
  const float* src = o + (size_t)w * d.dv;
  float ss = 0.f;
  for (int c = lane; c < d.dv; c += 32) ss = fmaf(src[c], src[c], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)d.dv + d.eps);
  const float* gate = proj + (size_t)t * ld + gate_off + (size_t)h * d.dv;
  for (int c = lane; c < d.dv; c += 32)
    elem<OT>::store(out + (size_t)w * d.dv + c, src[c] * inv * d.out_norm[c] * silu_f(gate[c]));
}

static bool delta_ok(const pieh_delta* d) {
  return d && d->H > 0 && d->G > 0 && d->H % d->G == 0 && d->dk > 0 && d->dv > 0 && d->taps >= 1 && d->taps <= kMaxTaps &&
         d->dk <= 512 && d->dv <= 512;
}

}  // namespace pieh

using namespace pieh;

extern "C" int pieh_delta_prepare(float* q, float* k, float* v, float* beta, float* decay, const float* proj, long long ld,
                                  const pieh_delta* d, const pieh_batch* b, void* stream) {
  if (!q || !k || !v || !beta || !decay || !proj || !d || !b) return PIE_ENULL;
  if (!delta_ok(d)) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  count_launch(2);
  launch_k(delta_prepare_kernel, dim3(b->T, 2 * d->G + d->H), dim3(128), 0, st, q, k, v, beta, decay, proj, ld, *d, *b);
  if (d->taps > 1) {
    const int C = 2 * d->G * d->dk + d->H * d->dv;
    launch_k(conv_advance_kernel, dim3((C + 127) / 128, b->n_seq), dim3(128), 0, st, proj, ld, *d, *b);
  }
  return status_of(cudaGetLastError());
}

extern "C" int pieh_delta_scan(float* o, const float* q, const float* k, const float* v, const float* beta,
                               const float* decay, const pieh_delta* d, const pieh_batch* b, void* stream) {
  if (!o || !q || !k || !v || !beta || !decay || !d || !b) return PIE_ENULL;
  if (!delta_ok(d)) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  // 16 rows of a state column per lane.  Measured on a 4096-row portion (dk = dv = 128, 16 heads, one sequence):
  // 8 rows per lane (16 lanes, 4 shuffle steps) 2.10 ms, 16 rows 1.74 ms, 32 rows (4 lanes, 2 steps, 64 CTAs) 2.62 ms
  constexpr int RPT = 16;
  int R = 1;
  while (R * RPT < d->dk) R <<= 1;   // lanes per column, a power of two <= 32
  const int cols = kScanThreads / R;
  const size_t smem = (size_t)2 * kScanChunk * (2 * d->dk + cols + 2) * 4;
  static bool opted = false;
  if (smem > 48 * 1024 && !opted) {
    cudaFuncSetAttribute(delta_scan_kernel<RPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    opted = true;
  }
  count_launch();
  return status_of(launch_k(delta_scan_kernel<RPT>, dim3((d->dv + cols - 1) / cols, d->H, b->n_seq), dim3(kScanThreads), smem,
                            (cudaStream_t)stream, o, q, k, v, beta, decay, *d, *b, R));
}

extern "C" int pieh_delta_gate(void* out, int out_dtype, const float* o, const float* proj, long long ld,
                               long long gate_off, const pieh_delta* d, int T, void* stream) {
  if (!out || !o || !proj || !d) return PIE_ENULL;
  if (!delta_ok(d)) return PIE_EINVAL_SHAPE;
  if (T == 0) return PIE_OK;
  const long long warps = (long long)T * d->H;
  count_launch();
  PIEH_DISPATCH_DTYPE(out_dtype, OT, launch_k(delta_gate_kernel<OT>, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, (OT*)out, o, proj, ld, gate_off, *d, T));
  return status_of(cudaGetLastError());
}
