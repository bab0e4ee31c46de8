// Parameter block shared by the sparse attention kernels.
#pragma once

#include "common.cuh"

namespace mxb {

struct SparseParams {
  const void* q;
  int64_t q_sb, q_sh, q_st;
  const void* comp_kv;
  const __half* comp_scales;
  const int64_t* comp_row_start;
  const int32_t* comp_row_count;
  int64_t n_comp;
  const void* raw_kv;
  const __half* raw_scales;
  int32_t raw_cap, raw_start;
  const int32_t* topk;
  int32_t k;
  const float* sinks;
  void* out;
  int64_t o_sb, o_sh, o_st;
  float* partial_ml;   // external partial mode
  float* ws_o;         // [nsplit][N][Dv]
  float* ws_ml;        // [nsplit][N][2]
  int32_t B, T, H, Dqk, Dv;
  float scale;
  int64_t pos0;
  const int64_t* pos0_dev;
  int32_t window, ratio;
  int32_t nsplit;
  int32_t* status;
  int32_t q_tma;      // q reaches shared memory by TMA (tensor map beside these parameters) instead of registers
  int32_t q_axis[3];  // which of (0 = head, 1 = token, 2 = batch) lies on dimensions 1..3 of that map
  int32_t cta_base;        // set by the tensor-core launcher: (token, split) index of this launch's CTA 0
  int32_t cluster_merge;   // set by the tensor-core launcher: the splits of a token ran as one thread-block cluster
                           // and merged through shared memory (no partials in the workspace, no merge kernel)
};

// tcgen05 path (16-bit / int8 KV).  Returns MXB_ERR_UNSUPPORTED when the shape is outside its range.
bool sparse_tc_eligible(int kv_dtype, int q_dtype, int H, int Dqk, int Dv);
int sparse_tc_splits(int B, int T, int H, int k, int raw_cap, int requested);
int launch_sparse_tc(SparseParams& p, int kv_dtype, int q_dtype, int out_dtype, cudaStream_t st);

}  // namespace mxb
