// Learned absolute positions and the post-norm residual.
//   embed_positions_kernel   x[t] = table[token] + pos_table[position]; also the act-dtype copy the first sublayer reads
//   postnorm_add_kernel      x[t] += rms_norm(y[t]) * w, where y is a sublayer's output: the sublayer read x itself, and
//                            its output passes through the norm on its way INTO the residual.  y is either a plain row or
//                            gathered here from a mixture of experts (weighted rows of the grouped down projection plus
//                            the gated shared expert), so the mixture's sum never goes through memory.
// One CTA per token row; the row of y stays in shared memory between the two passes.
#include "hyb_common.cuh"

namespace pieh {

template <typename ET, typename AT>
__global__ void embed_positions_kernel(float* x, AT* act, const ET* table, const ET* pos_table, const int32_t* tokens,
                                       const int32_t* positions, int W, int vocab, int max_pos) {
  pdl_sync();
  const int t = blockIdx.x;
  int id = tokens[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const ET* row = table + (size_t)id * W;
  const ET* prow = nullptr;
  if (pos_table) {
    int p = positions[t];
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
    prow = pos_table + (size_t)p * W;
  }
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = elem<ET>::load(row + c);
    if (prow) v += elem<ET>::load(prow + c);
    x[(size_t)t * W + c] = v;
    if (act) elem<AT>::store(act + (size_t)t * W + c, v);
  }
}

template <typename AT>
__global__ void __launch_bounds__(256) postnorm_add_kernel(float* x, AT* act, const float* y, const pieh_mix_sum mix,
                                                           const float* norm_w, float eps, int W) {
  extern __shared__ float row[];
  __shared__ float red[33];
  pdl_sync();
  const int t = blockIdx.x;
  float ss = 0.f;
  if (mix.parts) {
    float sg = 0.f;
    if (mix.shared) sg = 1.f / (1.f + expf(-mix.shared_gate[(size_t)t * mix.gate_ld]));
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      float v = 0.f;
      for (int k = 0; k < mix.top; ++k)   // fixed order: the sum does not depend on how the slots were handed out
        v = fmaf(mix.part_w[(size_t)t * mix.top + k], mix.parts[(size_t)mix.part_row[(size_t)t * mix.top + k] * W + c], v);
      if (mix.shared) v = fmaf(sg, mix.shared[(size_t)t * W + c], v);
      row[c] = v;
      ss = fmaf(v, v, ss);
    }
  } else {
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float v = y[(size_t)t * W + c];
      row[c] = v;
      ss = fmaf(v, v, ss);
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = x[(size_t)t * W + c] + row[c] * inv * norm_w[c];
    x[(size_t)t * W + c] = v;
    if (act) elem<AT>::store(act + (size_t)t * W + c, v);
  }
}

}  // namespace pieh

using namespace pieh;

extern "C" int pieh_embed_positions(float* x, void* act, int act_dtype, const void* table, const void* pos_table,
                                    int table_dtype, const int32_t* tokens, const int32_t* positions, int T, int W, int vocab,
                                    int max_positions, void* stream) {
  if (!x || !table || !tokens || (pos_table && !positions)) return PIE_ENULL;
  if (T < 0 || W < 1 || vocab < 1 || (pos_table && max_positions < 1)) return PIE_EINVAL_SHAPE;
  if (T == 0) return PIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  count_launch();
  PIEH_DISPATCH_DTYPE(table_dtype, ET, PIEH_DISPATCH_DTYPE(act_dtype, AT,
      launch_k(embed_positions_kernel<ET, AT>, dim3(T), dim3(256), 0, st, x, (AT*)act, (const ET*)table, (const ET*)pos_table,
               tokens, positions, W, vocab, max_positions)));
  return status_of(cudaGetLastError());
}

extern "C" int pieh_postnorm_add(float* x, void* act, int act_dtype, const float* y, const pieh_mix_sum* mix,
                                 const float* norm_w, float eps, int T, int W, void* stream) {
  if (!x || !norm_w || (!y && !(mix && mix->parts))) return PIE_ENULL;
  if (mix && mix->parts && (!mix->part_row || !mix->part_w || mix->top < 1 || (mix->shared && !mix->shared_gate)))
    return PIE_ENULL;
  if (T < 0 || W < 1 || (size_t)W * 4 > 200 * 1024) return PIE_EINVAL_SHAPE;
  if (T == 0) return PIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  pieh_mix_sum m = {};
  if (mix && mix->parts) m = *mix;
  const size_t smem = (size_t)W * 4;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(postnorm_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(postnorm_add_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  count_launch();
  PIEH_DISPATCH_DTYPE(act_dtype, AT, launch_k(postnorm_add_kernel<AT>, dim3(T), dim3(256), smem, st, x, (AT*)act, y, m, norm_w, eps, W));
  return status_of(cudaGetLastError());
}
