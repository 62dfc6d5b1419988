// Differential attention over 64-token pages, ragged steps.  A query head carries TWO maps (two query / key vectors of d
// features) over the same values:  o = unit_rms(softmax(s1) V - lambda softmax(s2) V) * out_scale,
// s = softcap * tanh(q . k * scale / softcap), keys visible inside a sliding window that ends at the query's own position.
// attn_prepare_kernel  per token: RMS norm of every (head, map) of q and k with a shared plain weight, rotation of adjacent
//                      feature pairs of the first rot_dims features (angle = position x frequency, evaluated in double),
//                      k and v written to the sequence's page at the token's position
// attn_run_kernel      one CTA per (token, query head): 8 warps take 32-key blocks of the window in turn, a lane scores
//                      one key for both maps, the warp keeps an online softmax per map and accumulates p V with the lanes
//                      spread over the value features; the warps merge through shared memory
// attn_tile_kernel     prompt portions over bf16 pages: 64-row query tiles on mma.sync (below)
// A step's keys are appended before its queries run, so a prompt portion sees itself through the same pages as its past.
#include "hyb_common.cuh"

namespace pieh {

constexpr int kPage = 64;

template <typename KT>
__global__ void __launch_bounds__(128) attn_prepare_kernel(float* q_out, const float* proj, long long ld, const pieh_attn a,
                                                           const pieh_batch b) {
  extern __shared__ float cs[];   // [rot_dims / 2][2]: cos, sin of this token's angles
  pdl_sync();
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

constexpr int kRunWarps = 8;

template <typename T> struct kv8;   // 8 consecutive cache elements as floats
template <> struct kv8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct kv8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
};

template <typename KT, typename OT, int NV>
__global__ void __launch_bounds__(kRunWarps * 32) attn_run_kernel(OT* out, const float* q, const pieh_attn a,
                                                                  const pieh_batch b) {
  extern __shared__ __align__(16) float sm[];
  __shared__ float red[33];
  constexpr int NW = kRunWarps, NTH = kRunWarps * 32;
  pdl_sync();
  const int t = blockIdx.x / a.H, h = blockIdx.x - t * a.H;
  const int g = h / (a.H / a.G);
  const int i = b.tok_seq[t], p = b.tok_pos[t];
  const int d = a.d, dv = a.dv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = sm;                  // [2][d]
  float* mg = qs + 2 * d;          // [warps][2 maps][dv + 2]: acc, m, l
  for (int c = threadIdx.x; c < 2 * d; c += NTH) qs[c] = q[((size_t)t * a.H + h) * 2 * d + c];
  __syncthreads();
  const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
  const int32_t* table = b.block_table + (size_t)i * b.bt_stride;
  const KT* kpool = reinterpret_cast<const KT*>(a.k_pages);
  const KT* vpool = reinterpret_cast<const KT*>(a.v_pages);
  const bool vec = (d & 7) == 0;   // rows of 2 d elements then start on 16-byte boundaries
  float m1 = -1e30f, m2 = -1e30f, l1 = 0.f, l2 = 0.f, acc1[NV], acc2[NV];
#pragma unroll
  for (int x = 0; x < NV; ++x) acc1[x] = acc2[x] = 0.f;
  for (int base = lo + warp * 32; base <= p; base += NW * 32) {
    const int j = base + lane;
    const bool ok = j <= p;
    long long slot = 0;
    float s1 = -1e30f, s2 = -1e30f;
    if (ok) {
      slot = (long long)table[j / kPage] * kPage + j % kPage;
      const KT* kr = kpool + ((size_t)slot * a.G + g) * 2 * d;
      float d1 = 0.f, d2 = 0.f;
      if (vec) {
#pragma unroll 4
        for (int c = 0; c < d; c += 8) {
          float k1[8], k2[8];
          kv8<KT>::load(kr + c, k1);
          kv8<KT>::load(kr + d + c, k2);
#pragma unroll
          for (int e = 0; e < 8; ++e) { d1 = fmaf(qs[c + e], k1[e], d1); d2 = fmaf(qs[d + c + e], k2[e], d2); }
        }
      } else {
        for (int c = 0; c < d; ++c) {
          d1 = fmaf(qs[c], elem<KT>::load(kr + c), d1);
          d2 = fmaf(qs[d + c], elem<KT>::load(kr + d + c), d2);
        }
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
    // all 32 keys of the block, four at a time with their loads issued together: a key past the row's position has
    // weight 0 and slot 0 (a valid, finite row), so it adds nothing
#pragma unroll 1
    for (int k0 = 0; k0 < 32; k0 += 4) {
      if (base + k0 > p) break;
      float w1[4], w2[4], vv[4][NV];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        w1[u] = __shfl_sync(0xffffffffu, p1, k0 + u);
        w2[u] = __shfl_sync(0xffffffffu, p2, k0 + u);
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
        for (int x = 0; x < NV; ++x) {
          acc1[x] = fmaf(w1[u], vv[u][x], acc1[x]);
          acc2[x] = fmaf(w2[u], vv[u][x], acc2[x]);
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
  // feature c = threadIdx.x (dv <= 256 = threads): merge the warps' partial softmaxes, combine the maps
  const int c = threadIdx.x;
  float ov = 0.f;
  if (c < dv) {
    float res[2];
    for (int mp = 0; mp < 2; ++mp) {
      float M = -1e30f;
      for (int w = 0; w < NW; ++w) M = fmaxf(M, mg[(size_t)(w * 2 + mp) * (dv + 2) + dv]);
      float L = 0.f, A = 0.f;
      for (int w = 0; w < NW; ++w) {
        const float* src = mg + (size_t)(w * 2 + mp) * (dv + 2);
        const float f = expf(src[dv] - M);
        L = fmaf(src[dv + 1], f, L);
        A = fmaf(src[c], f, A);
      }
      res[mp] = A / L;
    }
    ov = res[0] - a.lambda * res[1];
  }
  const float ssq = block_sum(ov * ov, red);
  const float inv = a.out_scale / sqrtf(ssq / (float)dv + a.eps);
  if (c < dv) elem<OT>::store(out + ((size_t)t * a.H + h) * dv + c, ov * inv);
}

// ---- prompt portions on the tensor cores ---------------------------------------------------------------------------
// A CTA of 4 warps owns one 64-row query tile (consecutive positions of ONE sequence) of one query head; key tiles are
// whole pages (64 keys) from the first page the window reaches to the page of the tile's last row, double-buffered in
// XOR-swizzled shared memory by cp.async.  Per map: S = Q_m K_m^T on mma.sync.m16n8k16 (bf16 in, fp32 out), scale,
// soft cap, causal and window mask, online softmax in fp32 (exp2 domain), P rounded to bf16, O_m += P V.  Both maps walk
// the same V tile.  The end combines the maps, normalises each row over its dv values and stores bf16.
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
template <int ROWB>   // bytes of a tile row; 16-byte chunk c of row r sits at chunk c ^ (r & 7)
__device__ __forceinline__ uint32_t tile_off(int r, int c) { return (uint32_t)(r * ROWB + ((c ^ (r & 7)) << 4)); }

template <int D, int DV>
__global__ void __launch_bounds__(128) attn_tile_kernel(__nv_bfloat16* out, const float* q, const pieh_attn a,
                                                        const pieh_batch b) {
  constexpr int KC = D / 16, NT = 8, DT = DV / 8;
  constexpr int KROWB = 2 * D * 2, VROWB = DV * 2;
  constexpr int KTILE = 64 * KROWB, VTILE = 64 * VROWB;
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_sync();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int tile = blockIdx.x, h = blockIdx.y;
  const int i = b.tile_seq[tile], row0 = b.tile_row[tile];
  const int nrows = min(64, b.seq_start[i] + b.seq_len[i] - row0);
  const int pos0 = b.tok_pos[row0];
  const int kvh = h / (a.H / a.G);
  const int last_key = pos0 + nrows - 1;
  const int first_key = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  const int j_lo = first_key / kPage, j_hi = last_key / kPage;
  const int32_t* table = b.block_table + (size_t)i * b.bt_stride;
  const __nv_bfloat16* kpool = reinterpret_cast<const __nv_bfloat16*>(a.k_pages);
  const __nv_bfloat16* vpool = reinterpret_cast<const __nv_bfloat16*>(a.v_pages);
  const uint32_t sK = (uint32_t)__cvta_generic_to_shared(smem), sV = sK + 2 * KTILE;

  auto issue = [&](int j) {
    const size_t page = (size_t)table[j] * kPage;
    const uint32_t dk = sK + ((j - j_lo) & 1) * KTILE, dvv = sV + ((j - j_lo) & 1) * VTILE;
    constexpr int CK = KROWB / 16, CV = VROWB / 16;
    for (int e = tid; e < 64 * CK; e += 128) {
      const int r = e / CK, c = e - r * CK;
      cp16(dk + tile_off<KROWB>(r, c), kpool + ((page + r) * a.G + kvh) * (2 * D) + c * 8);
    }
    for (int e = tid; e < 64 * CV; e += 128) {
      const int r = e / CV, c = e - r * CV;
      cp16(dvv + tile_off<VROWB>(r, c), vpool + ((page + r) * a.G + kvh) * DV + c * 8);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  issue(j_lo);

  // Q fragments of both maps: rows 16 warp + g and + 8 of the tile (rows past the tile's end repeat its last row)
  const int r0 = warp * 16 + g, r1 = r0 + 8;
  uint32_t qf[2][KC][4];
#pragma unroll
  for (int mp = 0; mp < 2; ++mp) {
    const float* q0 = q + (((size_t)(row0 + min(r0, nrows - 1)) * a.H + h) * 2 + mp) * D;
    const float* q1 = q + (((size_t)(row0 + min(r1, nrows - 1)) * a.H + h) * 2 + mp) * D;
#pragma unroll
    for (int kc = 0; kc < KC; ++kc) {
      const float2 x0 = *reinterpret_cast<const float2*>(q0 + kc * 16 + 2 * t4);
      const float2 x1 = *reinterpret_cast<const float2*>(q1 + kc * 16 + 2 * t4);
      const float2 x2 = *reinterpret_cast<const float2*>(q0 + kc * 16 + 8 + 2 * t4);
      const float2 x3 = *reinterpret_cast<const float2*>(q1 + kc * 16 + 8 + 2 * t4);
      qf[mp][kc][0] = pack2(x0.x, x0.y); qf[mp][kc][1] = pack2(x1.x, x1.y);
      qf[mp][kc][2] = pack2(x2.x, x2.y); qf[mp][kc][3] = pack2(x3.x, x3.y);
    }
  }
  float o[2][DT][4];
#pragma unroll
  for (int mp = 0; mp < 2; ++mp)
#pragma unroll
    for (int x = 0; x < DT; ++x) o[mp][x][0] = o[mp][x][1] = o[mp][x][2] = o[mp][x][3] = 0.f;
  float mrun[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}}, lrun[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  const int p0 = pos0 + min(r0, nrows - 1), p1 = pos0 + min(r1, nrows - 1);   // positions of this thread's two rows
  const int w0 = a.window > 0 ? p0 - a.window + 1 : 0, w1 = a.window > 0 ? p1 - a.window + 1 : 0;
  constexpr float kLog2e = 1.4426950408889634f;

  for (int j = j_lo; j <= j_hi; ++j) {
    if (j < j_hi) { issue(j + 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
    else asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const uint32_t tk = sK + ((j - j_lo) & 1) * KTILE, tv = sV + ((j - j_lo) & 1) * VTILE;
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
      float s[NT][4];
#pragma unroll
      for (int n = 0; n < NT; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
      for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int kc = 0; kc < KC; kc += 2) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(tk + tile_off<KROWB>(n * 8 + (lane & 7), mp * (D / 8) + kc * 2 + (lane >> 3)), b0, b1, b2, b3);
          mma_16816(s[n], qf[mp][kc][0], qf[mp][kc][1], qf[mp][kc][2], qf[mp][kc][3], b0, b1);
          mma_16816(s[n], qf[mp][kc + 1][0], qf[mp][kc + 1][1], qf[mp][kc + 1][2], qf[mp][kc + 1][3], b2, b3);
        }
      }
      const int key0 = j * kPage + 2 * t4;
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int k = key0 + n * 8;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[n][e] * a.scale;
          if (a.softcap > 0.f) v = a.softcap * (1.f - __fdividef(2.f, __expf(2.f * v / a.softcap) + 1.f));   // tanh, abs error ~1e-7
          const int key = k + (e & 1), pr = e < 2 ? p0 : p1, wl = e < 2 ? w0 : w1;
          s[n][e] = (key <= pr && key >= wl) ? v * kLog2e : -INFINITY;
        }
        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      if (mx0 > mrun[mp][0]) {
        const float c = exp2f(mrun[mp][0] - mx0);   // running maximum -inf: 0, and everything it multiplies is 0
        lrun[mp][0] *= c;
#pragma unroll
        for (int x = 0; x < DT; ++x) { o[mp][x][0] *= c; o[mp][x][1] *= c; }
        mrun[mp][0] = mx0;
      }
      if (mx1 > mrun[mp][1]) {
        const float c = exp2f(mrun[mp][1] - mx1);
        lrun[mp][1] *= c;
#pragma unroll
        for (int x = 0; x < DT; ++x) { o[mp][x][2] *= c; o[mp][x][3] *= c; }
        mrun[mp][1] = mx1;
      }
      const float ms0 = mrun[mp][0] == -INFINITY ? 0.f : mrun[mp][0], ms1 = mrun[mp][1] == -INFINITY ? 0.f : mrun[mp][1];
      float ps0 = 0.f, ps1 = 0.f;
      uint32_t pf[NT][2];
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const float e0 = exp2f(s[n][0] - ms0), e1 = exp2f(s[n][1] - ms0);
        const float e2 = exp2f(s[n][2] - ms1), e3 = exp2f(s[n][3] - ms1);
        ps0 += e0 + e1; ps1 += e2 + e3;
        pf[n][0] = pack2(e0, e1);
        pf[n][1] = pack2(e2, e3);
      }
      lrun[mp][0] += ps0; lrun[mp][1] += ps1;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint32_t a0 = pf[2 * kk][0], a1 = pf[2 * kk][1], a2 = pf[2 * kk + 1][0], a3 = pf[2 * kk + 1][1];
#pragma unroll
        for (int dj = 0; dj < DT; dj += 2) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_trans(tv + tile_off<VROWB>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dj + (lane >> 4)), b0, b1, b2, b3);
          mma_16816(o[mp][dj], a0, a1, a2, a3, b0, b1);
          mma_16816(o[mp][dj + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    __syncthreads();   // the stage is refilled two iterations from now
  }
  // ---- combine the maps, unit rms over the row's dv values, store --------------------------------------------------
  float inv[2][2];
#pragma unroll
  for (int mp = 0; mp < 2; ++mp)
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      float l = lrun[mp][rr];
      l += __shfl_xor_sync(0xffffffffu, l, 1); l += __shfl_xor_sync(0xffffffffu, l, 2);
      inv[mp][rr] = 1.f / l;
    }
  float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
  for (int x = 0; x < DT; ++x) {
    o[0][x][0] = o[0][x][0] * inv[0][0] - a.lambda * o[1][x][0] * inv[1][0];
    o[0][x][1] = o[0][x][1] * inv[0][0] - a.lambda * o[1][x][1] * inv[1][0];
    o[0][x][2] = o[0][x][2] * inv[0][1] - a.lambda * o[1][x][2] * inv[1][1];
    o[0][x][3] = o[0][x][3] * inv[0][1] - a.lambda * o[1][x][3] * inv[1][1];
    ss0 += o[0][x][0] * o[0][x][0] + o[0][x][1] * o[0][x][1];
    ss1 += o[0][x][2] * o[0][x][2] + o[0][x][3] * o[0][x][3];
  }
  ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1); ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
  ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1); ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
  const float n0 = a.out_scale / sqrtf(ss0 / (float)DV + a.eps), n1 = a.out_scale / sqrtf(ss1 / (float)DV + a.eps);
#pragma unroll
  for (int x = 0; x < DT; ++x) {
    const int c = x * 8 + 2 * t4;
    if (r0 < nrows) *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r0) * a.H + h) * DV + c) = pack2(o[0][x][0] * n0, o[0][x][1] * n0);
    if (r1 < nrows) *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r1) * a.H + h) * DV + c) = pack2(o[0][x][2] * n1, o[0][x][3] * n1);
  }
}

template <int D, int DV>
static cudaError_t launch_tile(__nv_bfloat16* out, const float* q, const pieh_attn& a, const pieh_batch& b, cudaStream_t st) {
  constexpr int smem = 2 * (64 * 2 * D * 2 + 64 * DV * 2);
  static unsigned long long configured = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(configured >> (dev & 63) & 1)) {
    cudaError_t e = cudaFuncSetAttribute(attn_tile_kernel<D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured |= 1ull << (dev & 63);
  }
  return launch_k(attn_tile_kernel<D, DV>, dim3(b.n_tiles, a.H), dim3(128), smem, st, out, q, a, b);
}

// the tile kernel serves steps that are mostly prompt portions, over bf16 pages, at the head sizes it is built for
static bool tile_ok(const pieh_attn& a, const pieh_batch& b, int out_dtype) {
  static const bool off = [] { const char* e = getenv("PIE_HYBRID_NO_TILE_ATTN"); return e && e[0] == '1'; }();
  return !off && a.kv_dtype == PIE_DTYPE_BF16 && out_dtype == PIE_DTYPE_BF16 && (a.d == 32 || a.d == 64) &&
         (a.dv == 64 || a.dv == 128) && b.n_tiles > 0 && b.tile_seq && b.tile_row && a.H <= 65535 &&
         (long long)b.T >= 16LL * b.n_seq;
}

static bool attn_ok(const pieh_attn* a) {
  return a && a->H > 0 && a->G > 0 && a->H % a->G == 0 && a->d > 0 && a->dv > 0 && a->dv <= 256 && a->d <= 1024 &&
         a->rot_dims >= 0 && a->rot_dims <= a->d && a->rot_dims % 2 == 0 && (a->rot_dims == 0 || a->rot_freqs) &&
         a->k_pages && a->v_pages && ((a->q_norm == nullptr) == (a->k_norm == nullptr));
}

template <typename KT, typename OT>
static cudaError_t launch_run(OT* out, const float* q, const pieh_attn& a, const pieh_batch& b, cudaStream_t st) {
  const size_t smem = ((size_t)2 * a.d + 2 * kRunWarps * (a.dv + 2)) * 4;
  const unsigned grid = (unsigned)b.T * a.H;
  const int nv = (a.dv + 31) / 32, nth = kRunWarps * 32;
  if (nv <= 1) return launch_k(attn_run_kernel<KT, OT, 1>, dim3(grid), dim3(nth), smem, st, out, q, a, b);
  if (nv <= 2) return launch_k(attn_run_kernel<KT, OT, 2>, dim3(grid), dim3(nth), smem, st, out, q, a, b);
  if (nv <= 4) return launch_k(attn_run_kernel<KT, OT, 4>, dim3(grid), dim3(nth), smem, st, out, q, a, b);
  return launch_k(attn_run_kernel<KT, OT, 8>, dim3(grid), dim3(nth), smem, st, out, q, a, b);
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
  PIEH_DISPATCH_DTYPE(a->kv_dtype, KT, launch_k(attn_prepare_kernel<KT>, dim3(b->T), dim3(128), smem, (cudaStream_t)stream, q_out, proj, ld, *a, *b));
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
  if (tile_ok(*a, *b, out_dtype)) {
    if (a->d == 32) e = a->dv == 64 ? launch_tile<32, 64>((bf*)out, q, *a, *b, st) : launch_tile<32, 128>((bf*)out, q, *a, *b, st);
    else e = a->dv == 64 ? launch_tile<64, 64>((bf*)out, q, *a, *b, st) : launch_tile<64, 128>((bf*)out, q, *a, *b, st);
    return status_of(e);
  }
  if (a->kv_dtype == PIE_DTYPE_BF16)
    e = out_dtype == PIE_DTYPE_BF16 ? launch_run<bf, bf>((bf*)out, q, *a, *b, st) : launch_run<bf, float>((float*)out, q, *a, *b, st);
  else
    e = out_dtype == PIE_DTYPE_BF16 ? launch_run<float, bf>((bf*)out, q, *a, *b, st) : launch_run<float, float>((float*)out, q, *a, *b, st);
  return status_of(e);
}
