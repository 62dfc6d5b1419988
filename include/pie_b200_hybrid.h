/* pie_b200_hybrid.h -- C ABI of libpie_b200_hybrid.so: sm_100a operators for models that mix recurrent and attention
 * layers over dense (unquantized) weights.  Built from csrc/hyb_*.cu; the page allocator of pie_b200.h is linked in too,
 * so a program that serves such a model needs this one library only.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer; calls are asynchronous on `stream` (cudaStream_t as void*), allocate nothing,
 *     never synchronise and can be captured in CUDA graphs; the return value is a pie_status (pie_b200.h);
 *   - a step is RAGGED: T token rows, row t belongs to sequence tok_seq[t]; sequence i owns rows
 *     seq_start[i] .. seq_start[i] + seq_len[i] - 1 (consecutive positions seq_ctx[i] ..), keeps its recurrent state in
 *     slot seq_slot[i] and its keys / values in the 64-token pages named by row i of the block table;
 *   - dtype codes are PIE_DTYPE_BF16 / PIE_DTYPE_F32.  "act" tensors (inputs of matrix products, the key / value pages)
 *     are bf16 when the model is served in bf16 and fp32 when it runs in exact mode; the residual streams, norms,
 *     softmax, recurrent state and every gate of a recurrence are fp32 in both;
 *   - small parameters (norm weights, mixing weights, convolution taps, decay parameters) are fp32 arrays.
 */
#ifndef PIE_B200_HYBRID_H_
#define PIE_B200_HYBRID_H_

#include <stddef.h>
#include <stdint.h>

#include "pie_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

int pieh_abi_version(void);
const char* pieh_last_cuda_error(void);
unsigned long long pieh_launch_count(void);
/* non-zero after a tensor-core pipeline gave up a bounded wait (the kernel returned early; its output is invalid).
 * Synchronises the device. */
unsigned int pieh_pipeline_error(void);
/* on: every operator is launched as a programmatic dependent of the launch before it on its stream (its blocks may become
 * resident early and wait at their top); captured into CUDA graphs as such.  Off by default. */
void pieh_set_pdl(int on);

/* epilogues of pieh_linear */
enum {
  PIEH_EPI_NONE = 0,
  PIEH_EPI_RELU2 = 1,    /* y <- max(y, 0)^2                                   */
  PIEH_EPI_SOFTCAP = 2,  /* y <- cap * tanh(y / cap)                           */
  PIEH_EPI_STREAMS = 3   /* out is the residual [M, S, N] fp32: x[m, t, n] <- sum_s mix[s, t] x[m, s, n] + outw[t] * y */
};

/* ragged step descriptor, shared by the recurrent and the attention operators (all arrays int32, device) */
typedef struct pieh_batch {
  int T;                   /* token rows in the step                          */
  int n_seq;               /* sequences in the step                           */
  const int32_t* tok_seq;  /* [T]      sequence index of each row             */
  const int32_t* tok_pos;  /* [T]      position of each row in its sequence   */
  const int32_t* seq_start;/* [n_seq]  first row of the sequence              */
  const int32_t* seq_len;  /* [n_seq]  rows of the sequence in this step      */
  const int32_t* seq_ctx;  /* [n_seq]  tokens of the sequence before this step*/
  const int32_t* seq_slot; /* [n_seq]  state slot of the sequence             */
  const int32_t* block_table; /* [n_seq, bt_stride] page ids                  */
  int bt_stride;
  int n_tiles;             /* 64-row query tiles: every sequence's rows cut into runs of <= 64 (0: no tile list)  */
  const int32_t* tile_seq; /* [n_tiles] sequence of the tile                  */
  const int32_t* tile_row; /* [n_tiles] first row of the tile                 */
} pieh_batch;

/* y[m, n] = sum_k x[m, k] w[n, k] (+ bias[n]), fp32 accumulation.  w_dtype bf16: x is rounded to bf16 (if it is not
 * already) and the products are exact; w_dtype f32: plain fp32 multiply-add, no reduced-precision matrix mode.
 * bias fp32 or NULL.  epi_a: cap (SOFTCAP); STREAMS: out_ld = S * N is implied, mix [S, S] and outw [S] fp32, S <= 8. */
int pieh_linear(void* out, int out_dtype, long long out_ld, const void* x, int x_dtype, long long x_ld, const void* w,
                int w_dtype, const float* bias, int M, int N, int K, int epilogue, float epi_a, const float* mix,
                const float* outw, int S, void* stream);

/* xs[t, s, :] = table[tokens[t], :] for every stream s.  xs fp32 [T, S, W]. */
int pieh_embed_streams(float* xs, const void* table, int table_dtype, const int32_t* tokens, int T, int S, int W,
                       int vocab, void* stream);
/* out[r, :] = rms_norm(sum_s in_w[s] xs[row(r), s, :]) * (unit_offset + norm_w);  in_w NULL = all ones; rows NULL =
 * identity.  out is an act tensor [R, W]. */
int pieh_stream_norm(void* out, int out_dtype, const float* xs, const int32_t* rows, const float* in_w,
                     const float* norm_w, float unit_offset, float eps, int R, int S, int W, void* stream);
/* xs[t, u, :] <- sum_s mix[s, u] xs[t, s, :] + outw[u] * y[t, :]   (y fp32 [T, W]) */
int pieh_stream_update(float* xs, const float* y, const float* mix, const float* outw, int T, int S, int W, void* stream);

/* ---- gated delta rule ----------------------------------------------------------------------------------------------
 * proj fp32 [T, ld]: columns [q (G dk) | k (G dk) | v (H dv) | gate (H dv) | b (H) | a (H)] of the fused projection. */
typedef struct pieh_delta {
  int H, G, dk, dv, taps;
  const float* conv_w;   /* [(2 G dk + H dv), taps]; last tap multiplies the current token */
  const float* A_log;    /* [H] */
  const float* dt_bias;  /* [H] */
  const float* out_norm; /* [dv] */
  float eps;             /* of the output norm */
  float* conv_state;     /* [slots, taps - 1, 2 G dk + H dv] fp32, oldest first */
  float* state;          /* [slots, H, dk, dv] fp32 */
} pieh_delta;
/* convolution + silu, unit-length q (times dk^-1/2) and k, beta and decay per head; then the convolution history of
 * every sequence moves on.  q, k fp32 [T, G, dk]; v fp32 [T, H, dv]; beta, decay fp32 [T, H]. */
int pieh_delta_prepare(float* q, float* k, float* v, float* beta, float* decay, const float* proj, long long ld,
                       const pieh_delta* d, const pieh_batch* b, void* stream);
/* the recurrence over each sequence's rows, state read from and written back to its slot (a sequence with no context
 * starts from zero whatever the slot holds); o fp32 [T, H, dv]. */
int pieh_delta_scan(float* o, const float* q, const float* k, const float* v, const float* beta, const float* decay,
                    const pieh_delta* d, const pieh_batch* b, void* stream);
/* out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * out_norm * silu(gate[t, h, :]); gate = proj + gate_off, row stride ld */
int pieh_delta_gate(void* out, int out_dtype, const float* o, const float* proj, long long ld, long long gate_off,
                    const pieh_delta* d, int T, void* stream);

/* ---- differential attention with a sliding window over 64-token pages ----------------------------------------------
 * proj fp32 [T, ld]: columns [q (H, 2, d) | k (G, 2, d) | v (G, dv)]. */
typedef struct pieh_attn {
  int H, G, d, dv;
  int rot_dims;            /* leading features of each map that rotate (adjacent pairs); 0 = none */
  const double* rot_freqs; /* [rot_dims / 2] angle per position */
  const float* q_norm;     /* [d] plain weight, or NULL = no query / key norm */
  const float* k_norm;
  float eps;
  float scale, softcap;    /* softcap 0 = none */
  int window;              /* visible keys per query (itself included); 0 = all earlier ones */
  float lambda;            /* weight of the second map */
  float out_scale;         /* applied after the per-head unit-rms of (map1 - lambda map2) */
  void* k_pages;           /* [pages, 64, G, 2 d] act dtype */
  void* v_pages;           /* [pages, 64, G, dv]  act dtype */
  int kv_dtype;
} pieh_attn;
/* norm + rotation of q and k; k and v appended to the pages at each row's position.  q_out fp32 [T, H, 2, d]. */
int pieh_attn_prepare(float* q_out, const float* proj, long long ld, const pieh_attn* a, const pieh_batch* b,
                      void* stream);
/* out[t, h, :] act [T, H dv]: both maps' windowed softmax attention over the pages, combined and normalised. */
int pieh_attn_run(void* out, int out_dtype, const float* q, const pieh_attn* a, const pieh_batch* b, void* stream);

#ifdef __cplusplus
}
#endif
#endif
