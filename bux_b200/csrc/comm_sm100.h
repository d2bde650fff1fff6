// Launchers of the expert-parallel exchange kernels (comm_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace bux {

struct Status;

void ep_push_rows(const void* x, const int* src_token, const int* dst_rank, const int* dst_row,
                  const float* row_scale, const uint64_t* peer_base, const uint64_t* peer_scale, long picks, int d,
                  int sms, cudaStream_t s);
// token by token, the rows quantised on the way (MXFP8 along the row): token t's row goes to row
// row_of[t, j] of rank rank_of[t, j] for each of its k picks (row < 0: dropped), e4m3 bytes into
// peer_q[rank] ([cap, d]), E8M0 scales row-major into peer_sf[rank] ([cap, d/32] bytes), w[t, j]
// (1 without w) into peer_scale[rank][row] when given; d % 128 == 0, k <= 32
void ep_push_rows_mx(const void* x, const int* rank_of, const int* row_of, const float* w, const uint64_t* peer_q,
                     const uint64_t* peer_sf, const uint64_t* peer_scale, long tokens, int k, int d, int sms,
                     cudaStream_t s);
// out[r] = <a[r], b[r]> over rows of d bf16
void row_dots(const void* a, const void* b, float* out, long rows, int d, cudaStream_t s);
// out[i] = peer[rank_of[i]][row_of[i]] (fp32), after the peers' flags reached `epoch`
void ep_pull_scalar(const uint64_t* peer_base, const int* rank_of, const int* row_of, float* out, long picks,
                    const int* flags, int world, int epoch, uint64_t limit_ns, Status* st, cudaStream_t s);
void ep_signal(const uint64_t* peer_flags, int channel, int world, int my_rank, int epoch, cudaStream_t s);
void ep_pull_combine(const uint64_t* peer_base, const int* rank_of, const int* row_of, const float* w, void* out,
                     long tokens, int k, int d, const int* flags, int world, int epoch, uint64_t limit_ns,
                     Status* st, cudaStream_t s);
void ep_pull_dot(const uint64_t* peer_base, const int* rank_of, const int* row_of, const void* dout, float* dw,
                 long picks, int k, int d, cudaStream_t s);
void zero_pad_rows(void* buf, const int* offsets, const int* counts, int groups, int d, cudaStream_t s);
void tp_push_block(const void* src, const uint64_t* peer_base, int world, int my_rank, long rows, int d, int sms,
                   cudaStream_t s);
void tp_pull_reduce(const uint64_t* peer_base, int world, int my_rank, long rows, int d, void* out,
                    const void* residual, const int* flags, int epoch, uint64_t limit_ns, Status* st,
                    cudaStream_t s);
// row-major E8M0 scales [rows, sf_cols] (sf_cols % 4 == 0) -> the GEMM's 512-byte scale tiles
void sf_rows_to_tiles(const void* src, void* dst, long rows, int sf_cols, cudaStream_t s);
void set_comm_ctas_per_sm(int n);  // 0: each kernel's own default
void ep_wait(const int* flags, int world, int epoch, uint64_t limit_ns, Status* st, cudaStream_t s);

}  // namespace bux
