// Residual streams (hyper-connections): S fp32 copies of the residual per token, xs [T, S, W].  A sublayer reads a
// weighted sum of the streams through an RMS norm (stream_norm) and writes back by mixing the streams and adding its
// output to each with its own weight (stream_update; pieh_linear's STREAMS epilogue does the same inside the
// output projection).  S = 1 with unit weights is the ordinary pre-norm residual.
#include <atomic>
#include <cstdio>

#include "hyb_common.cuh"

namespace pieh {

static std::atomic<unsigned long long> g_launches{0};
static thread_local char g_err[256] = "";
static std::atomic<int> g_pdl{0};
bool pdl_enabled() { return g_pdl.load(std::memory_order_relaxed) != 0; }
void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }
int status_of(cudaError_t e) {
  if (e == cudaSuccess) return PIE_OK;
  snprintf(g_err, sizeof(g_err), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
  return PIE_ECUDA;
}
int num_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <typename ET>
__global__ void embed_streams_kernel(float* xs, const ET* table, const int32_t* tokens, int S, int W, int vocab) {
  pdl_sync();
  const int t = blockIdx.x;
  int id = tokens[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const ET* row = table + (size_t)id * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = elem<ET>::load(row + c);
    for (int s = 0; s < S; ++s) xs[((size_t)t * S + s) * W + c] = v;
  }
}

// one CTA per output row; the combined row is kept in shared memory between the two passes (W floats)
template <typename OT>
__global__ void stream_norm_kernel(OT* out, const float* xs, const int32_t* rows, const float* in_w, const float* norm_w,
                                   float unit_offset, float eps, int S, int W) {
  extern __shared__ float row[];
  __shared__ float red[33];
  pdl_sync();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  const float* src = xs + (size_t)t * S * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float u = 0.f;
    for (int s = 0; s < S; ++s) u = fmaf(in_w ? in_w[s] : 1.f, src[(size_t)s * W + c], u);
    row[c] = u;
    ss = fmaf(u, u, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x)
    elem<OT>::store(out + (size_t)r * W + c, row[c] * inv * (unit_offset + norm_w[c]));
}

__global__ void stream_update_kernel(float* xs, const float* y, const float* mix, const float* outw, int S, int W,
                                     long long n) {
  pdl_sync();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // over T * W
  if (i >= n) return;
  const long long t = i / W;
  const int c = (int)(i - t * W);
  float* p = xs + (size_t)t * S * W + c;
  float old[8];
  for (int s = 0; s < S; ++s) old[s] = p[(size_t)s * W];
  const float yv = y[i];
  for (int u = 0; u < S; ++u) {
    float acc = outw[u] * yv;
    for (int s = 0; s < S; ++s) acc = fmaf(mix[s * S + u], old[s], acc);
    p[(size_t)u * W] = acc;
  }
}

}  // namespace pieh

using namespace pieh;

extern "C" int pieh_abi_version(void) { return 1; }
extern "C" const char* pieh_last_cuda_error(void) { return g_err; }
extern "C" unsigned long long pieh_launch_count(void) { return g_launches.load(); }
extern "C" void pieh_set_pdl(int on) { g_pdl.store(on ? 1 : 0); }

extern "C" int pieh_embed_streams(float* xs, const void* table, int table_dtype, const int32_t* tokens, int T, int S, int W,
                                  int vocab, void* stream) {
  if (!xs || !table || !tokens) return PIE_ENULL;
  if (T < 0 || S < 1 || W < 1 || vocab < 1) return PIE_EINVAL_SHAPE;
  if (T == 0) return PIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  count_launch();
  PIEH_DISPATCH_DTYPE(table_dtype, ET, launch_k(embed_streams_kernel<ET>, dim3(T), dim3(256), 0, st, xs, (const ET*)table, tokens, S, W, vocab));
  return status_of(cudaGetLastError());
}

extern "C" int pieh_stream_norm(void* out, int out_dtype, const float* xs, const int32_t* rows, const float* in_w,
                                const float* norm_w, float unit_offset, float eps, int R, int S, int W, void* stream) {
  if (!out || !xs || !norm_w) return PIE_ENULL;
  if (R < 0 || S < 1 || W < 1 || (size_t)W * 4 > 200 * 1024) return PIE_EINVAL_SHAPE;
  if (R == 0) return PIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)W * 4;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(stream_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(stream_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  count_launch();
  PIEH_DISPATCH_DTYPE(out_dtype, OT, launch_k(stream_norm_kernel<OT>, dim3(R), dim3(256), smem, st, (OT*)out, xs, rows, in_w, norm_w, unit_offset, eps, S, W));
  return status_of(cudaGetLastError());
}

extern "C" int pieh_stream_update(float* xs, const float* y, const float* mix, const float* outw, int T, int S, int W,
                                  void* stream) {
  if (!xs || !y || !mix || !outw) return PIE_ENULL;
  if (T < 0 || S < 1 || S > 8 || W < 1) return PIE_EINVAL_SHAPE;
  if (T == 0) return PIE_OK;
  const long long n = (long long)T * W;
  count_launch();
  launch_k(stream_update_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, xs, y, mix, outw, S, W, n);
  return status_of(cudaGetLastError());
}
