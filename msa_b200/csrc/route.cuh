// Declarations shared by the routing translation units.
#pragma once
#include "common.cuh"

namespace msa {

constexpr int kRouteMaxN = 256;  // widest query tile (UMMA N) of the tensor-core kernel

int reset_score_table(uint32_t* keys, int64_t table_stride, int32_t n_cols, int32_t n_seq, float min_val,
                      cudaStream_t stream);

int launch_route_simt(int32_t dtype, const void* qf, const float* row_bias, int n_seq, int s_pad, const void* rk,
                      int64_t rk_stride, int n_chunks, int kdim, const int32_t* chunk_doc, int n_docs, float alpha,
                      uint32_t* keys, int64_t table_stride, int32_t* status, cudaStream_t stream);

int launch_route_tc(const void* qf, const float* row_bias, int n_seq, int s_pad, const void* rk, int64_t rk_stride,
                    int n_chunks, int kdim, const int32_t* chunk_doc, int n_docs, float alpha, float min_val,
                    uint32_t* keys, int64_t table_stride, int32_t* status, bool blocked, cudaStream_t stream);

}  // namespace msa
