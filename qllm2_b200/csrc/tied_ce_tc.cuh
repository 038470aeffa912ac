// Interface between the cross-entropy host code and its tensor-core (tcgen05) kernels.
#pragma once
#include "common.cuh"

namespace qpam {

struct CETcPlan {
  bool enabled;          // bf16 inputs with 16-byte aligned rows
  int32_t n_tiles;       // vocabulary tiles of 256 columns
  int32_t nsplit;        // vocabulary splits of the statistics pass (grid.x)
  int32_t tiles_per_split;
  int64_t chunk_rows;    // rows per backward chunk (multiple of 128)
  int32_t ksplit;        // split-K factor of the dH GEMM
  int32_t dw_bufs;       // fp32 [V][F] accumulation buffers of dW (one per row chunk, at most 4; 0 for a single chunk)
};

CETcPlan ce_tc_plan(const qpam_ce_args* a);

struct CETcBuffers {
  float *pm, *ps, *pt, *pbest;
  int32_t* pidx;
  void* pbuf;       // bf16 [chunk_rows][ldp]
  int64_t ldp;
  float* dh_part;   // [ksplit][chunk_rows][F]
  float* dwacc;     // [dw_bufs][V][F]
};

// per-row partial statistics [nsplit][N] via the tensor-core logits GEMM
int ce_tc_partial(const qpam_ce_args* a, const CETcPlan& plan, const CETcBuffers& b, cudaStream_t st);
// out[N][ld] (bf16) = h w^T through the same GEMM, tiles stored by TMA (ld a multiple of 8, out 16-byte aligned)
int ce_tc_logits(const qpam_ce_args* a, const CETcPlan& plan, void* out, int64_t ld, cudaStream_t st);
// dH, dW via recomputed probabilities (bf16 tiles) and two tensor-core GEMMs per row chunk
// dh_ready_stream (may be NULL): a stream of the caller that is made to wait until dh is complete, while the
// dw products continue on `st`
int ce_tc_backward(const qpam_ce_args* a, const CETcPlan& plan, const CETcBuffers& b, const float* lse,
                   const float* grad_scale, const float* denom, void* dh, void* dw, cudaStream_t st,
                   cudaStream_t dh_ready_stream);
int signal_stream(cudaStream_t st, cudaStream_t waiter);

// device error word of the tensor-core kernels (0 = ok; 101..104 = a bounded wait gave up)
int ce_tc_device_status(int* value, bool clear);

}  // namespace qpam
