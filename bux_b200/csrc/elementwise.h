// Launchers of the memory-bound kernels (elementwise.cu). Pointers are device
// pointers; none of these functions allocates or synchronises.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace bux {

enum { ACT_SWISH = 0, ACT_QUICK_GELU = 1, ACT_GELU_TANH = 2, ACT_RELU2 = 3, ACT_IDENTITY = 4 };
enum { MOM_F32 = 0, MOM_BF16 = 1, MOM_FP8 = 2 };

void rmsnorm_fwd(const void* x, const float* w, void* y, float* rstd, long rows, int d, float eps, cudaStream_t s);
void rmsnorm_bwd(const void* x, const float* w, const void* dy, const float* rstd, void* dx, float* dw, long rows, int d, cudaStream_t s);
const char* norm_rope(bool bwd, const void* x, const float* w, const float* cs, const float* sn, void* y,
                      float* rstd, const void* dy, float* dw, long tokens, int heads, int D,
                      long stride_x, long stride_y, float eps, cudaStream_t s);
void glu_fwd(const void* h, void* out, const float* row_scale, long rows, int f, int kind, float limit, float up_offset, cudaStream_t s);
void glu_bwd(const void* h, const void* dout, void* dh, const float* row_scale, float* d_row_scale, long rows, int f, int kind, float limit, float up_offset, cudaStream_t s);
void quant_mxfp8(const void* x, long ld_x, const int* row_index, const float* row_scale, uint8_t* q_row, uint8_t* sf_row, uint8_t* q_col, uint8_t* sf_col, long rows, int cols, long ld_col, int batch, long x_batch_stride, cudaStream_t s);
// Quantise glu(h) [rows, f] (dout null) or the gradient of h [rows, 2f] given dout [rows, f],
// computed tile by tile from h [rows, 2f]; f % 128 == 0 for the gradient. `row_scale` (fp32
// [rows], activation only) multiplies row r of the activation before it is rounded.
void quant_mxfp8_glu(const void* h, const void* dout, const float* row_scale, uint8_t* q_row, uint8_t* sf_row,
                     uint8_t* q_col, uint8_t* sf_col, long rows, int f, long ld_col, int kind, float limit,
                     float up_offset, cudaStream_t s);
// The transposed MXFP8 copy ([cols, ld_col], quantised along the rows) of a matrix that is
// already MXFP8 along its columns (e4m3 bytes [rows, cols] + scale tiles): dequantise, requantise.
void requant_mxfp8_cols(const uint8_t* q, const uint8_t* sf, uint8_t* q_col, uint8_t* sf_col, long rows, int cols,
                        long ld_col, cudaStream_t s);
// NVFP4 along the rows: E2M1 codes two per byte [rows, cols / 2], E4M3 scale bytes [rows, cols / 16]
void quant_nvfp4(const void* x, const float* tensor_scale, uint8_t* packed, uint8_t* scales, long rows, int cols,
                 cudaStream_t s);
void ce_fwd_bwd(void* logits, const int* targets, const float* mask, float* loss, float* logz, long rows, int vocab, long ld, float grad_scale, float z_weight, float softcap, cudaStream_t s);
const char* adamw(void* p, bool p_bf16, const void* g, bool g_bf16, void* m, void* v, uint8_t* m_sf, uint8_t* v_sf, int mom,
                  void* shadow, long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                  const float* gscale_ptr, float gscale, cudaStream_t s);
void sumsq(const void* g, bool bf16, long n, float* out, cudaStream_t s);
// indices (int64) of the k largest entries of each fp32 row, descending; n <= 512
const char* topk_rows(const float* scores, long* idx, long rows, int n, int k, cudaStream_t s);
void gather_rows(const void* x, const int* index, void* out, long rows, int d, cudaStream_t s);
void combine_bwd(const void* y, const void* dout, const int* pos, const float* w, void* dy, float* dw, long picks, int k, int d, cudaStream_t s);
// causal depthwise convolution over the tokens (conv_sm100.cu): forward (bwd = false: out = y, `in` = x) and
// the input gradient (bwd = true: out = dx, `in` = dy); w [C, taps] fp32, position [B, T] int32 or null
const char* causal_conv(bool bwd, const void* in, const float* w, const float* bias, const int* position, void* out,
                        int B, int T, int C, int taps, cudaStream_t s);
// dw [C, taps] and db [C] (or null), fp32, ADDED to what they hold
const char* causal_conv_wgrad(const void* x, const void* dy, const int* position, float* dw, float* db, int B, int T,
                              int C, int taps, cudaStream_t s);
void combine_rows(const void* y, const int* pos, const float* w, void* out, long tokens, int k, int d, cudaStream_t s);

}  // namespace bux
