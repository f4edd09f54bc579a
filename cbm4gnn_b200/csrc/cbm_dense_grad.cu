// Gradients of the dense maps of the GCN layers (see cbm_dense.cu): input gradient dX = dY W and weight
// gradient dW = dY^T X as fp32-accurate tensor-core GEMMs.
#include "cbm_dense_gemm.cuh"

namespace cbm_dense {

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

using GemmNN = FastGemm<RowMajor, RowMajor, 128, 16>;   // A K-contiguous, B N-contiguous: dY W
using GemmNN64 = FastGemm<RowMajor, RowMajor, 64, 32>;
using GemmNNMask = FastGemm<RowMajor, RowMajor, 128, 16, false, true>;  // dY W, zeroed where the ReLU output is 0
using GemmNN64Mask = FastGemm<RowMajor, RowMajor, 64, 32, false, true>;
using GemmTN = FastGemm<ColMajor, RowMajor, 128, 16>;   // A M-contiguous, B N-contiguous: dY^T X
using GemmTN64 = FastGemm<ColMajor, RowMajor, 64, 32>;

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

extern "C" int cbm_b200_dense_grad_input(const float* dy, int64_t lddy, const float* w, int64_t ldw, float* dx,
                                         int64_t lddx, int32_t n_rows, int32_t n_in, int32_t n_out, void* stream) {
    if (!dy || !w || !dx || n_rows < 0 || n_in <= 0 || n_out <= 0)
        return cbm::fail(CBM_B200_ERR_ARG, "dense_grad_input: bad arguments");
    if (n_rows == 0) return CBM_B200_OK;
    return run_either<GemmNN, GemmNN64>(n_in, "dense_grad_input", n_rows, n_in, n_out, 1, dy, lddy, (int64_t)0, w, ldw,
                                        (int64_t)0, dx, lddx, (int64_t)0, (void*)nullptr, (size_t)0, (cudaStream_t)stream);
}

extern "C" int cbm_b200_dense_grad_input_relu(const float* dy, int64_t lddy, const float* w, int64_t ldw, const float* h,
                                              int64_t ldh, float* dx, int64_t lddx, int32_t n_rows, int32_t n_in,
                                              int32_t n_out, void* stream) {
    if (!dy || !w || !h || !dx || n_rows < 0 || n_in <= 0 || n_out <= 0)
        return cbm::fail(CBM_B200_ERR_ARG, "dense_grad_input_relu: bad arguments");
    if (ldh < n_in || ldh % 4 != 0 || (reinterpret_cast<uintptr_t>(h) & 15) != 0)
        return cbm::fail(CBM_B200_ERR_ARG, "dense_grad_input_relu: h must have 16-byte aligned rows of at least n_in floats");
    if (n_rows == 0) return CBM_B200_OK;
    return run_either<GemmNNMask, GemmNN64Mask>(n_in, "dense_grad_input_relu", n_rows, n_in, n_out, 1, dy, lddy, (int64_t)0, w,
                                                ldw, (int64_t)0, dx, lddx, (int64_t)0, (void*)nullptr, (size_t)0,
                                                (cudaStream_t)stream, h, ldh);
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
