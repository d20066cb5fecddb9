// Interface of the tcgen05 implicit-GEMM engine (tc_gemm.cu).
#pragma once

#include "common.cuh"

namespace pdnn {

// True if the tensor-core engine can run this convolution pass (channel/feature alignment for
// TMA, strides 1 or 2, at most 64 filter taps, NHWC, groups == 1, 16-byte aligned pointers).
bool tc_conv_supported(int pass, int dtype, const void* in, const void* fil, const void* out,
                       const PdnnConv2DParams& p);

// Scratch elements (of dtype) the pass needs: only the filter backprop's split reduction uses any.
size_t tc_conv_workspace_elems(int pass, int dtype, const PdnnConv2DParams& p);

// Returned by tc_conv2d when the tensor maps of a few-channel layer could not be encoded: the caller
// runs the layer on the direct kernel instead.
constexpr int kNeedsDirect = -1;

int tc_conv2d(int pass, int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams& p,
              const PdnnConvEpilogue* epi, const PdnnBackpropFusion* fusion, void* ws, size_t ws_elems, cudaStream_t s);

// Grouped forward convolution with STRIDED groups whose per-group channel and feature counts meet
// tc_conv_supported's alignment rules: one implicit GEMM per group on channel slices of the tensors.
bool tc_grouped_conv_supported(int dtype, const void* in, const void* fil, const void* out, const PdnnConv2DParams& p);
int tc_grouped_conv_forward(int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams& p,
                            const PdnnConvEpilogue* epi, cudaStream_t s);

bool tc_matmul_supported(int dtype, int tl, int tr, const void* lhs, const void* rhs, const void* out, int batches,
                         int m, int k, int n);
// out_f32: the product is written as fp32 whatever dtype is (beta then scales fp32 values).
int tc_matmul(int dtype, int tl, int tr, const void* lhs, const void* rhs, void* out, int batches, int m, int k, int n,
              float beta, cudaStream_t s, bool out_f32 = false);

// General CUDA-core matmul for shapes the tensor-core engine cannot take.
int simt_matmul(int dtype, int tl, int tr, const void* lhs, const void* rhs, void* out, int batches, int m, int k, int n,
                float beta, cudaStream_t s, bool out_f32 = false);

// Copies the device-side error record (4 words; word 0 == 0 means no error) to the host.
// Synchronises the device.
int tc_read_error_record(unsigned out[4], int clear);

}  // namespace pdnn
