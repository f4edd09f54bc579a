// Dense maps of the GCN layers on the 5th-generation tensor cores (sm_100a).
//
// A GCN layer of the reference is `lin` followed by `propagate`
// (gnns/graph_convolutional_network/cbm_gcn.py:21-24): a bias-free [N,in] x [in,out] map in fp32.
// The sparse half runs in cbm_engine.cu; this file is the dense half and its two gradients
//     forward   Y  = X  W^T      X [N,in],   W [out,in]          -> Y  [N,out]
//     input     dX = dY W        dY [N,out], W [out,in]          -> dX [N,in]
//     weight    dW = dY^T X      dY [N,out], X [N,in]            -> dW [out,in]
// as fp32-accurate GEMMs on tcgen05: every fp32 operand is split on the fly into three bf16 terms
// (x = b0 + b1 + b2 with 8 mantissa bits each), the products of the terms that matter are issued as
// bf16 UMMA instructions with TMA-staged operands and accumulated in fp32 in tensor memory.  The
// result carries fp32 accuracy (error ~2^-22 relative per product), which the 1e-4 tolerance of the
// reference's tests needs and single-pass TF32/BF16 does not give.
//
// The kernels are instantiations of the CUTLASS sm100 collective builders (TMA loads without
// cluster multicast — cluster shape 1x1x1 —, an input-transform warp group, tcgen05.mma with the
// accumulator in TMEM, TMA-store epilogue).  The weight gradient contracts over the N rows of the
// graph (hundreds of thousands) into a tiny [out,in] result, so it runs as a batched GEMM over row
// chunks followed by a reduction of the partial results in a fixed order.
#include "cbm_dense_gemm.cuh"

namespace cbm_dense {
// wide (128-column) and narrow (64-column) result tiles; A and B K-contiguous: X W^T
using GemmNT = FastGemm<RowMajor, ColMajor, 128, 16>;
using GemmNT64 = FastGemm<RowMajor, ColMajor, 64, 32>;
using GemmNTRelu = FastGemm<RowMajor, ColMajor, 128, 16, true>;
using GemmNT64Relu = FastGemm<RowMajor, ColMajor, 64, 32, true>;
}  // namespace cbm_dense

using namespace cbm_dense;

extern "C" int cbm_b200_dense_forward(const float* x, int64_t ldx, const float* w, int64_t ldw, float* y, int64_t ldy,
                                      int32_t n_rows, int32_t n_in, int32_t n_out, void* stream) {
    if (!x || !w || !y || n_rows < 0 || n_in <= 0 || n_out <= 0)
        return cbm::fail(CBM_B200_ERR_ARG, "dense_forward: bad arguments");
    if (n_rows == 0) return CBM_B200_OK;
    return run_either<GemmNT, GemmNT64>(n_out, "dense_forward", n_rows, n_out, n_in, 1, x, ldx, (int64_t)0, w, ldw,
                                        (int64_t)0, y, ldy, (int64_t)0, (void*)nullptr, (size_t)0, (cudaStream_t)stream);
}

extern "C" int cbm_b200_dense_forward_relu(const float* x, int64_t ldx, const float* w, int64_t ldw, float* y,
                                           int64_t ldy, int32_t n_rows, int32_t n_in, int32_t n_out, void* stream) {
    if (!x || !w || !y || n_rows < 0 || n_in <= 0 || n_out <= 0)
        return cbm::fail(CBM_B200_ERR_ARG, "dense_forward_relu: bad arguments");
    if (n_rows == 0) return CBM_B200_OK;
    return run_either<GemmNTRelu, GemmNT64Relu>(n_out, "dense_forward_relu", n_rows, n_out, n_in, 1, x, ldx, (int64_t)0, w,
                                                ldw, (int64_t)0, y, ldy, (int64_t)0, (void*)nullptr, (size_t)0,
                                                (cudaStream_t)stream);
}

