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
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <string>

#include "cutlass/cutlass.h"
#include "cute/tensor.hpp"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/util/packed_stride.hpp"

#include "cbm_b200.h"
#include "cbm_common.h"

namespace cbm_dense {

using namespace cute;
using RowMajor = cutlass::layout::RowMajor;
using ColMajor = cutlass::layout::ColumnMajor;

// D[M,N] = A[M,K] * B[K,N], fp32 in and out, row-major D.  One CTA computes a 128 x TileN tile with
// the split A operand held in tensor memory where its layout allows (K-contiguous A), else in
// shared memory.  Measured on B200 (N = 235 868 rows): 128 x 128 x 16 tiles 0.20 ms for 128 -> 256 and
// 0.18 ms for 256 -> 128 (cuBLAS fp32 SIMT: 0.33 / 0.31 ms); a 64-column result takes 0.10 ms with
// 128 x 64 tiles against 0.18 ms with 128 x 128 tiles (half of every tile wasted).
template <class LayoutA, class LayoutB, int TileN, int TileK>
struct FastGemm {
    using TileShape = Shape<_128, Int<TileN>, Int<TileK>>;
    using ClusterShape = Shape<_1, _1, _1>;
    using CollectiveEpilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, TileShape, ClusterShape,
        cutlass::epilogue::collective::EpilogueTileAuto, float, float, float, RowMajor, 4, float, RowMajor, 4,
        cutlass::epilogue::TmaWarpSpecialized1Sm>::CollectiveOp;
    using CollectiveMainloop = typename cutlass::gemm::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, float, LayoutA, 4, float, LayoutB, 4, float, TileShape,
        ClusterShape,
        cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename CollectiveEpilogue::SharedStorage))>,
        cutlass::gemm::KernelTmaWarpSpecialized1SmFastFP32Sm100>::CollectiveOp;
    using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, CollectiveMainloop, CollectiveEpilogue, void>;
    using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;
    using StrideA = typename Kernel::StrideA;
    using StrideB = typename Kernel::StrideB;
    using StrideD = typename Kernel::StrideD;
};

template <class G>
int run_gemm(const char* who, int m, int n, int k, int batch, const float* a, int64_t lda, int64_t batch_a,
             const float* b, int64_t ldb, int64_t batch_b, float* d, int64_t ldd, int64_t batch_d, void* workspace,
             size_t workspace_bytes, cudaStream_t stream) {
    typename G::StrideA sa{};
    typename G::StrideB sb{};
    typename G::StrideD sd{};
    // the leading dimension sits in the non-unit mode of each stride, the batch stride in the last
    if constexpr (is_static_v<remove_cvref_t<decltype(get<0>(sa))>>) {
        get<1>(sa) = lda;  // A stored with M contiguous (column-major)
    } else {
        get<0>(sa) = lda;  // K contiguous (row-major)
    }
    if constexpr (is_static_v<remove_cvref_t<decltype(get<0>(sb))>>) {
        get<1>(sb) = ldb;  // N contiguous
    } else {
        get<0>(sb) = ldb;  // K contiguous
    }
    get<0>(sd) = ldd;
    get<2>(sa) = batch_a;
    get<2>(sb) = batch_b;
    get<2>(sd) = batch_d;
    typename G::Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm,
                                     {m, n, k, batch},
                                     {a, sa, b, sb},
                                     {{1.0f, 0.0f}, nullptr, sd, d, sd}};
    // The TMA descriptors are encoded through the driver API, which wants a context current on the
    // calling thread; a thread that has made no runtime call yet (an autograd worker) has none
    // until the device is set.
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess)
        return cbm::fail(CBM_B200_ERR_CUDA, std::string(who) + ": no usable CUDA device on this thread");
    try {
        typename G::Gemm gemm;
        if (gemm.can_implement(args) != cutlass::Status::kSuccess)
            return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": shape or alignment not supported (widths and leading "
                                                                  "dimensions must be multiples of 4 floats, pointers 16-byte aligned)");
        if (G::Gemm::get_workspace_size(args) > workspace_bytes)
            return cbm::fail(CBM_B200_ERR_ALLOC, std::string(who) + ": workspace too small");
        cutlass::Status st = gemm.initialize(args, workspace, stream);
        if (st == cutlass::Status::kSuccess) st = gemm.run(stream);
        if (st != cutlass::Status::kSuccess)
            return cbm::fail(CBM_B200_ERR_CUDA, std::string(who) + ": " + cutlassGetStatusString(st));
    } catch (const std::exception& e) {  // nothing may unwind through the C boundary
        return cbm::fail(CBM_B200_ERR_CUDA, std::string(who) + ": " + e.what());
    } catch (...) {
        return cbm::fail(CBM_B200_ERR_CUDA, std::string(who) + ": unknown failure in the GEMM set-up");
    }
    return CBM_B200_OK;
}

// fixed-order sum of `parts` partial [rows, cols] results (each a contiguous block) into out, which
// is [rows, cols] with leading dimension ldo, or its transpose [cols, rows] when `transpose`
__global__ void reduce_partials_kernel(const float* __restrict__ part, int parts, int64_t block, float* __restrict__ out,
                                       int rows, int cols, int64_t ldo, int transpose) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)rows * cols) return;
    float s = 0.f;
    for (int p = 0; p < parts; ++p) s += part[(int64_t)p * block + i];
    const int64_t r = i / cols, c = i % cols;
    out[transpose ? c * ldo + r : r * ldo + c] = s;
}

// wide (128-column) and narrow (64-column) result tiles for each operand layout
using GemmNT = FastGemm<RowMajor, ColMajor, 128, 16>;   // A K-contiguous, B K-contiguous: X W^T
using GemmNT64 = FastGemm<RowMajor, ColMajor, 64, 32>;
using GemmNN = FastGemm<RowMajor, RowMajor, 128, 16>;   // A K-contiguous, B N-contiguous: dY W
using GemmNN64 = FastGemm<RowMajor, RowMajor, 64, 32>;
using GemmTN = FastGemm<ColMajor, RowMajor, 128, 16>;   // A M-contiguous, B N-contiguous: dY^T X
using GemmTN64 = FastGemm<ColMajor, RowMajor, 64, 32>;

// columns of 128-wide tiles needed for n result columns against 64-wide ones
bool narrow_tiles_win(int n) { return ((n + 63) / 64) * 64 < ((n + 127) / 128) * 128; }

template <class Wide, class Narrow, class... Args>
int run_either(int n, Args... args) {
    return narrow_tiles_win(n) ? run_gemm<Narrow>(args...) : run_gemm<Wide>(args...);
}

// Row chunks for the weight gradient: as many as make the CTAs of one launch a whole number of
// waves over the SMs (result tiles x chunks = 2 x SM count), each a multiple of 16 rows.
int64_t weight_chunks(int32_t n_rows, int32_t m, int32_t n, bool narrow) {
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t tiles = (int64_t)((m + 127) / 128) * ((n + (narrow ? 63 : 127)) / (narrow ? 64 : 128));
    int64_t chunks = std::max<int64_t>(1, (2 * (int64_t)sms) / std::max<int64_t>(1, tiles));
    chunks = std::min<int64_t>(chunks, CBM_B200_DENSE_MAX_CHUNKS);
    chunks = std::min<int64_t>(chunks, std::max<int64_t>(1, n_rows / 256));  // at least 256 rows per chunk
    return chunks;
}

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

extern "C" int cbm_b200_dense_grad_input(const float* dy, int64_t lddy, const float* w, int64_t ldw, float* dx,
                                         int64_t lddx, int32_t n_rows, int32_t n_in, int32_t n_out, void* stream) {
    if (!dy || !w || !dx || n_rows < 0 || n_in <= 0 || n_out <= 0)
        return cbm::fail(CBM_B200_ERR_ARG, "dense_grad_input: bad arguments");
    if (n_rows == 0) return CBM_B200_OK;
    return run_either<GemmNN, GemmNN64>(n_in, "dense_grad_input", n_rows, n_in, n_out, 1, dy, lddy, (int64_t)0, w, ldw,
                                        (int64_t)0, dx, lddx, (int64_t)0, (void*)nullptr, (size_t)0, (cudaStream_t)stream);
}

extern "C" int64_t cbm_b200_dense_grad_weight_workspace(int32_t n_rows, int32_t n_in, int32_t n_out) {
    (void)n_rows;
    return (int64_t)(CBM_B200_DENSE_MAX_CHUNKS + 1) * n_in * n_out * (int64_t)sizeof(float);
}

// dW [out,in] = dY^T X.  The result is produced in whichever orientation wastes fewer tile columns
// — as dW (M = out, N = in) or as dW^T (M = in, N = out) — and the reduction of the partial results
// writes it out in [out,in] order either way.
extern "C" int cbm_b200_dense_grad_weight(const float* dy, int64_t lddy, const float* x, int64_t ldx, float* dw,
                                          int64_t lddw, int32_t n_rows, int32_t n_in, int32_t n_out, void* workspace,
                                          int64_t workspace_bytes, void* stream) {
    if (!dy || !x || !dw || n_rows < 0 || n_in <= 0 || n_out <= 0)
        return cbm::fail(CBM_B200_ERR_ARG, "dense_grad_weight: bad arguments");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t need = cbm_b200_dense_grad_weight_workspace(n_rows, n_in, n_out);
    if (!workspace || workspace_bytes < need)
        return cbm::fail(CBM_B200_ERR_ARG, "dense_grad_weight: workspace of " + std::to_string(need) + " bytes needed");
    auto padded = [](int m, int n) {  // elements computed, tile padding included
        const bool narrow = narrow_tiles_win(n);
        return (int64_t)((m + 127) / 128) * 128 * ((n + (narrow ? 63 : 127)) / (narrow ? 64 : 128)) * (narrow ? 64 : 128);
    };
    const bool transposed = padded(n_in, n_out) < padded(n_out, n_in);
    const int m = transposed ? n_in : n_out, n = transposed ? n_out : n_in;
    const float* a = transposed ? x : dy;
    const float* b = transposed ? dy : x;
    const int64_t lda = transposed ? ldx : lddy, ldb = transposed ? lddy : ldx;
    float* part = static_cast<float*>(workspace);
    const int64_t block = (int64_t)m * n;
    const int64_t chunks = weight_chunks(n_rows, m, n, narrow_tiles_win(n));
    const int64_t rows_per = (n_rows / chunks) / 16 * 16;
    int parts = 0;
    if (rows_per > 0) {
        int rc = run_either<GemmTN, GemmTN64>(n, "dense_grad_weight", m, n, (int)rows_per, (int)chunks, a, lda, rows_per * lda,
                                              b, ldb, rows_per * ldb, part, (int64_t)n, block, (void*)nullptr, (size_t)0, s);
        if (rc) return rc;
        parts = (int)chunks;
    }
    // The rows that do not fill the chunks (fewer than 16 per chunk) would be a long serial
    // contraction for the two or four CTAs of one more product; they are cut into 64-row pieces
    // contracted side by side, and what is left after those (< 64 rows) is one short product.
    int64_t done = rows_per > 0 ? rows_per * chunks : 0;
    const int64_t piece = 64;
    const int64_t n_pieces = std::min<int64_t>((n_rows - done) / piece, CBM_B200_DENSE_MAX_CHUNKS - parts - 1);
    if (n_pieces > 0) {
        int rc = run_either<GemmTN, GemmTN64>(n, "dense_grad_weight", m, n, (int)piece, (int)n_pieces, a + done * lda, lda,
                                              piece * lda, b + done * ldb, ldb, piece * ldb,
                                              part + (int64_t)parts * block, (int64_t)n, block, (void*)nullptr, (size_t)0, s);
        if (rc) return rc;
        parts += (int)n_pieces;
        done += piece * n_pieces;
    }
    if (done < n_rows) {
        int rc = run_either<GemmTN, GemmTN64>(n, "dense_grad_weight", m, n, (int)(n_rows - done), 1, a + done * lda, lda,
                                              (int64_t)0, b + done * ldb, ldb, (int64_t)0, part + (int64_t)parts * block,
                                              (int64_t)n, (int64_t)0, (void*)nullptr, (size_t)0, s);
        if (rc) return rc;
        ++parts;
    }
    reduce_partials_kernel<<<(unsigned)((block + 255) / 256), 256, 0, s>>>(part, parts, block, dw, m, n, lddw, transposed ? 1 : 0);
    if (cudaGetLastError() != cudaSuccess) return cbm::fail(CBM_B200_ERR_CUDA, "dense_grad_weight: reduction launch failed");
    return CBM_B200_OK;
}
