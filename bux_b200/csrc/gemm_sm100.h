// Host-visible types of the tcgen05 GEMM family (gemm_sm100.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bux {

struct Status;

enum { KIND_BF16 = 0, KIND_MXFP8 = 1 };
enum { MODE_DENSE = 0, MODE_GROUPED_ROWS = 1, MODE_GROUPED_K = 2 };
enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ACC = 2, OUT_BF16_ACC = 3 };  // *_ACC: C += A·B^T

// Kernel parameters (passed by value as a __grid_constant__).
struct GemmParams {
  alignas(64) CUtensorMap tmap_a;
  alignas(64) CUtensorMap tmap_b;
  alignas(64) CUtensorMap tmap_c;   // bf16 output as [32 rows x 64 columns] boxes (TMA-store epilogue)
  const uint8_t* sfa;        // MXFP8 scale tiles of A (512 bytes per 128 rows x 128 K)
  const uint8_t* sfb;
  void* c;
  const int* group_offsets;  // groups + 1 entries: row (or K) range of each group
  Status* status;
  int mode, M, N, K, k_total, groups, ldc, out_kind;
  // optional: before its first load the producer waits (bounded) until
  // wait_flags[0..wait_world) >= wait_epoch: senders on peer GPUs filled operand A
  const int* wait_flags; int wait_world, wait_epoch; unsigned long long wait_limit_ns;
  // wait_rows > 0: per-sender row blocks (see GemmArgs); m_rotate in tiles
  int wait_rows, m_rotate, wait_on_k, wait_on_n;
  int tma_store;  // the epilogue stages bf16 tiles in shared memory and stores them by TMA
};

// What a caller fills in. `a_outer/a_inner` are the stored dims of A (inner contiguous):
// [M, K] when K-major, [K, M] when MN-major; same for B with N.
struct GemmArgs {
  int kind = KIND_BF16, mode = MODE_DENSE, bn = 256, out_kind = OUT_BF16;
  bool a_mn = false, b_mn = false;
  const void* a = nullptr; uint64_t a_outer = 0, a_inner = 0, lda_bytes = 0;
  const void* b = nullptr; uint64_t b_outer = 0, b_inner = 0, ldb_bytes = 0;
  const uint8_t* sfa = nullptr; const uint8_t* sfb = nullptr;
  void* c = nullptr; int ldc = 0;
  int M = 0, N = 0, K = 0, k_total = 0, groups = 1;
  const int* group_offsets = nullptr;
  Status* status = nullptr;
  int sms = 0;
  const int* wait_flags = nullptr; int wait_world = 0, wait_epoch = 0;
  unsigned long long wait_limit_ns = 5000000000ull;
  // wait_rows > 0: the flagged operand arrives in blocks of wait_rows rows per sender
  // (rows of A, or of the contraction dimension with wait_on_k); a tile waits only for
  // the sender of its rows. m_rotate (dense mode, in tiles) starts the walk at this
  // rank's own rows, which need no wait.
  int wait_rows = 0, m_rotate = 0; bool wait_on_k = false;
  bool wait_on_n = false;  // the senders write row blocks of B (sharded weights arriving from their owners)
};

// Returns nullptr on success, else a static message.
const char* gemm_launch(const GemmArgs& args, cudaStream_t stream);
const char* make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows,
                         uint64_t cols, uint64_t row_stride_bytes, uint32_t box_cols,
                         uint32_t box_rows);

}  // namespace bux
