// Shared by cbm_dense.cu (forward maps) and cbm_dense_grad.cu (gradients): the fp32-accurate tensor-core
// GEMM as a CUTLASS sm100 instantiation and its launcher.  Two translation units so that the template
// instantiations, which dominate the build time, compile side by side.
#pragma once
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
// The collective builder fixes the number of computed bands (anti-diagonals i + j of the products
// a_i b_j of the three-term splits) at 5 = all 9 products.  Rebuilds its result with another count.
template <class Op, int Bands>
struct WithBands;
template <int L2T, int T2M, int Sch, int Acc, int NB, int SF, int API, class CS, class ACA, class Arch, class... Rest,
          int Bands>
struct WithBands<cutlass::gemm::collective::CollectiveMma<
                     cutlass::gemm::MainloopSm100TmaUmmaWarpSpecializedFastF32<L2T, T2M, Sch, Acc, NB, SF, API, CS, ACA, Arch>,
                     Rest...>,
                 Bands> {
    using type = cutlass::gemm::collective::CollectiveMma<
        cutlass::gemm::MainloopSm100TmaUmmaWarpSpecializedFastF32<L2T, T2M, Sch, Acc, Bands, SF, API, CS, ACA, Arch>, Rest...>;
};

// Three bands = the six products a_i b_j with i + j <= 2.  The three dropped ones are below 2^-24 of
// |a||b|; measured against float64 the result errs by 1.2e-7 of sum |a||b| (cuBLAS fp32: 4e-7), and a
// training step of the 2-layer GCN takes 1.58 ms instead of 1.61 ms with all nine.  128 x 128 x 32
// tiles (3 + 3 pipeline stages instead of 7 + 6) were measured 4 % slower than 128 x 128 x 16.
#ifndef CBM_DENSE_BANDS
#define CBM_DENSE_BANDS 3
#endif

template <class LayoutA, class LayoutB, int TileN, int TileK, bool Relu = false, bool MaskByAux = false>
struct FastGemm {
    static constexpr bool kMaskByAux = MaskByAux;
    using TileShape = Shape<_128, Int<TileN>, Int<TileK>>;
    using ClusterShape = Shape<_1, _1, _1>;
    // epilogue: D = acc; or D = max(acc, 0) for the map that feeds the ReLU between two layers; or
    // D = acc where a second row-major operand (the ReLU's output, loaded by TMA) is non-zero and 0
    // elsewhere, for the input gradient that flows back through that ReLU
    using Fusion = cute::conditional_t<
        MaskByAux,
        cutlass::epilogue::fusion::LinCombDeEltAct<RowMajor, cutlass::epilogue::thread::dReLU, float, float, float>,
        cute::conditional_t<Relu, cutlass::epilogue::fusion::LinCombEltAct<cutlass::epilogue::thread::ReLu, float, float>,
                            cutlass::epilogue::fusion::LinearCombination<float, float>>>;
    using CollectiveEpilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, TileShape, ClusterShape,
        cutlass::epilogue::collective::EpilogueTileAuto, float, float, float, RowMajor, 4, float, RowMajor, 4,
        cutlass::epilogue::TmaWarpSpecialized1Sm, Fusion>::CollectiveOp;
    using BuiltMainloop = typename cutlass::gemm::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, float, LayoutA, 4, float, LayoutB, 4, float, TileShape,
        ClusterShape,
        cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename CollectiveEpilogue::SharedStorage))>,
        cutlass::gemm::KernelTmaWarpSpecialized1SmFastFP32Sm100>::CollectiveOp;
    using CollectiveMainloop = typename WithBands<BuiltMainloop, CBM_DENSE_BANDS>::type;
    using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, CollectiveMainloop, CollectiveEpilogue, void>;
    using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;
    using StrideA = typename Kernel::StrideA;
    using StrideB = typename Kernel::StrideB;
    using StrideD = typename Kernel::StrideD;
};

template <class G>
int run_gemm(const char* who, int m, int n, int k, int batch, const float* a, int64_t lda, int64_t batch_a,
             const float* b, int64_t ldb, int64_t batch_b, float* d, int64_t ldd, int64_t batch_d, void* workspace,
             size_t workspace_bytes, cudaStream_t stream, const float* aux = nullptr, int64_t ldaux = 0) {
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
    if constexpr (G::kMaskByAux) {
        if (!aux) return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": mask operand is NULL");
        args.epilogue.thread.aux_ptr = aux;
        get<0>(args.epilogue.thread.dAux) = ldaux;
    }
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

// columns of 128-wide tiles needed for n result columns against 64-wide ones
inline bool narrow_tiles_win(int n) { return ((n + 63) / 64) * 64 < ((n + 127) / 128) * 128; }

template <class Wide, class Narrow, class... Args>
int run_either(int n, Args... args) {
    return narrow_tiles_win(n) ? run_gemm<Narrow>(args...) : run_gemm<Wide>(args...);
}

}  // namespace cbm_dense
