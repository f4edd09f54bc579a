// Candidate search of the CBM builder on the GPU.
//
// The builder's first step finds, for every row u, the rows v that share more than (|u| + alpha) / 2
// columns with it (the candidate rule of cbm/cbm_extensions.cpp:75-102, which the reference evaluates
// on all of A * A^T).  The host search (cbm_builder.cpp) walks, for every u, the column lists of u's
// rarest columns and counts hits per row; on a high-degree graph that is billions of random counter
// increments and 97 % of the build.  Here the same filter runs with one thread block per parent
// row: warps stream the column lists of the prefix and count with atomics into a per-block array of
// 16-bit counters that stays in L2, rows that reach the required number of hits get their exact
// intersection from a bitmap of u's columns, and survivors of the rule are appended to one output
// list.  The filter is lossless (see cbm_builder.cpp), so the set of candidates — and with it the
// structure the builder emits — is identical to the host search's; only the order of the output
// differs, and the caller sorts it.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "cbm_candidates.h"

namespace {

using i32 = int32_t;
using i64 = int64_t;
using u32 = uint32_t;
using u64 = unsigned long long;

struct SearchParams {
    i32 n, alpha;
    const i64* row_ptr;   // rows of the pattern, columns replaced by their rank (rare = small), ascending
    const i32* row_rank;
    const i32* col_of_rank;
    const i64* col_ptr;   // column lists (rows ascending), indexed by original column id
    const i32* col_rows;
    u32* hits;            // per block: (n + 1) / 2 words, two 16-bit counters each
    i32* touched;         // per block: n entries
    u32* bitmap;          // per block: (n + 31) / 32 words, bit per rank id
    i64 hits_stride, touched_stride, bitmap_stride;
    cbm::CandTriple* out;
    u64* out_count;       // [0] entries appended, [1] next parent row to claim
    i64 out_cap;
    i32* skipped;         // parents left to the host (prefix too long for 16-bit counters)
    i32* n_skipped;
};

constexpr int kThreads = 512;
constexpr int kMaxPrefix = 65000;

__global__ void __launch_bounds__(kThreads) candidate_kernel(const SearchParams p) {
    __shared__ i32 s_u, s_touched;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = kThreads / 32;
    u32* hits = p.hits + (i64)blockIdx.x * p.hits_stride;
    i32* touched = p.touched + (i64)blockIdx.x * p.touched_stride;
    u32* bitmap = p.bitmap + (i64)blockIdx.x * p.bitmap_stride;
    for (;;) {
        if (tid == 0) {
            s_u = (i32)atomicAdd(p.out_count + 1, 1ULL);
            s_touched = 0;
        }
        __syncthreads();
        const i32 u = s_u;
        if (u >= p.n) return;
        const i64 ub = p.row_ptr[u];
        const i32 nu = (i32)(p.row_ptr[u + 1] - ub);
        // shared columns an edge u -> v needs, and the prefix that guarantees j_hits of them
        const i64 sum = (i64)nu + p.alpha;
        const i64 half_floor = sum >= 0 ? sum / 2 : -((-sum + 1) / 2);
        const i64 need64 = max(half_floor + 1, (i64)1);
        bool skip = need64 > nu;
        const i32 need = (i32)min(need64, (i64)INT32_MAX);
        const i32 j_hits = min(need, max(8, min(32, need / 8)));
        const i32 plen = nu - need + j_hits;
        if (!skip && plen > kMaxPrefix) {
            if (tid == 0) p.skipped[atomicAdd(p.n_skipped, 1)] = u;
            skip = true;
        }
        if (skip) {
            __syncthreads();
            continue;
        }
        // 1. count hits of every row through the column lists of the prefix
        for (i32 i = warp; i < plen; i += n_warps) {
            const i32 c = p.col_of_rank[p.row_rank[ub + i]];
            const i64 qb = p.col_ptr[c], qe = p.col_ptr[c + 1];
            for (i64 q = qb + lane; q < qe; q += 32) {
                const i32 v = p.col_rows[q];
                const u32 old = atomicAdd(hits + (v >> 1), (v & 1) ? 0x10000u : 1u);
                if ((((v & 1) ? (old >> 16) : old) & 0xffffu) == 0) touched[atomicAdd(&s_touched, 1)] = v;
            }
        }
        const bool has_tail = plen < nu;
        if (has_tail)
            for (i32 i = tid; i < nu; i += kThreads) {
                const i32 r = p.row_rank[ub + i];
                atomicOr(bitmap + (r >> 5), 1u << (r & 31));
            }
        __syncthreads();
        // 2. rows with enough hits in the prefix: exact intersection, then the rule
        const i32 n_touched = s_touched;
        for (i32 t = warp; t < n_touched; t += n_warps) {
            const i32 v = touched[t];
            i32 in_prefix = 0;
            if (lane == 0) {
                const u32 w = atomicAnd(hits + (v >> 1), (v & 1) ? 0x0000ffffu : 0xffff0000u);  // read and clear
                in_prefix = (i32)(((v & 1) ? (w >> 16) : w) & 0xffffu);
            }
            in_prefix = __shfl_sync(0xffffffffu, in_prefix, 0);
            if (v == u || in_prefix < j_hits) continue;
            const i64 vb = p.row_ptr[v];
            const i32 nv = (i32)(p.row_ptr[v + 1] - vb);
            if (nv < need) continue;
            i32 both = in_prefix;
            if (has_tail) {
                i32 cnt = 0;
                for (i32 k = lane; k < nv; k += 32) {
                    const i32 r = p.row_rank[vb + k];
                    cnt += (i32)((bitmap[r >> 5] >> (r & 31)) & 1u);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
                both = cnt;
            }
            const i32 h = nu + nv - 2 * both;
            if (h < nv - p.alpha && lane == 0) {  // cbm/cbm_extensions.cpp:93-101
                const u64 pos = atomicAdd(p.out_count, 1ULL);
                if ((i64)pos < p.out_cap) p.out[pos] = cbm::CandTriple{u, v, h};
            }
        }
        __syncthreads();
        if (has_tail)
            for (i32 i = tid; i < nu; i += kThreads) bitmap[p.row_rank[ub + i] >> 5] = 0;
        __syncthreads();
    }
}

template <class T>
cudaError_t to_device(T** dst, const T* src, size_t count) {
    *dst = nullptr;
    cudaError_t e = cudaMalloc((void**)dst, std::max<size_t>(count, 1) * sizeof(T));
    if (e == cudaSuccess && count) e = cudaMemcpy(*dst, src, count * sizeof(T), cudaMemcpyHostToDevice);
    return e;
}

}  // namespace

namespace cbm {

int gpu_candidates(int device, int32_t n, int32_t alpha, const int64_t* row_ptr, const int32_t* row_rank,
                   const int32_t* col_of_rank, const int64_t* col_ptr, const int32_t* col_rows,
                   std::vector<CandTriple>& out, std::vector<int32_t>& left_to_host, std::string& err) {
    out.clear();
    left_to_host.clear();
    if (n <= 0) return 0;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) {
        err = std::string("gpu_candidates: cudaSetDevice: ") + cudaGetErrorString(e);
        return 1;
    }
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int blocks = (int)std::min<int64_t>((int64_t)sms * 2, n);
    const int64_t nnz = row_ptr[n];
    SearchParams p{};
    p.n = n;
    p.alpha = alpha;
    p.hits_stride = ((int64_t)n + 1) / 2 + 1;
    p.touched_stride = n;
    p.bitmap_stride = ((int64_t)n + 31) / 32 + 1;
    p.out_cap = std::max<int64_t>(8ll << 20, 16ll * n);
    i64* d_row_ptr = nullptr;
    i64* d_col_ptr = nullptr;
    i32 *d_row_rank = nullptr, *d_col_of_rank = nullptr, *d_col_rows = nullptr, *d_skipped = nullptr, *d_n_skipped = nullptr;
    u64* d_count = nullptr;
    auto cleanup = [&]() {
        cudaFree(d_row_ptr);
        cudaFree(d_col_ptr);
        cudaFree(d_row_rank);
        cudaFree(d_col_of_rank);
        cudaFree(d_col_rows);
        cudaFree(d_skipped);
        cudaFree(d_n_skipped);
        cudaFree(d_count);
        cudaFree(p.hits);
        cudaFree(p.touched);
        cudaFree(p.bitmap);
        cudaFree(p.out);
        if (prev >= 0) cudaSetDevice(prev);
    };
    auto fail = [&](const char* what, cudaError_t ce) {
        err = std::string("gpu_candidates: ") + what + ": " + cudaGetErrorString(ce);
        cleanup();
        return 1;
    };
    if ((e = to_device(&d_row_ptr, row_ptr, (size_t)n + 1)) != cudaSuccess) return fail("row_ptr", e);
    if ((e = to_device(&d_col_ptr, col_ptr, (size_t)n + 1)) != cudaSuccess) return fail("col_ptr", e);
    if ((e = to_device(&d_row_rank, row_rank, (size_t)nnz)) != cudaSuccess) return fail("row_rank", e);
    if ((e = to_device(&d_col_of_rank, col_of_rank, (size_t)n)) != cudaSuccess) return fail("col_of_rank", e);
    if ((e = to_device(&d_col_rows, col_rows, (size_t)nnz)) != cudaSuccess) return fail("col_rows", e);
    if ((e = cudaMalloc((void**)&d_skipped, (size_t)n * sizeof(i32))) != cudaSuccess) return fail("skipped", e);
    if ((e = cudaMalloc((void**)&d_n_skipped, sizeof(i32))) != cudaSuccess) return fail("n_skipped", e);
    if ((e = cudaMalloc((void**)&d_count, 2 * sizeof(u64))) != cudaSuccess) return fail("count", e);
    if ((e = cudaMalloc((void**)&p.hits, (size_t)blocks * p.hits_stride * sizeof(u32))) != cudaSuccess) return fail("hits", e);
    if ((e = cudaMalloc((void**)&p.touched, (size_t)blocks * p.touched_stride * sizeof(i32))) != cudaSuccess) return fail("touched", e);
    if ((e = cudaMalloc((void**)&p.bitmap, (size_t)blocks * p.bitmap_stride * sizeof(u32))) != cudaSuccess) return fail("bitmap", e);
    p.row_ptr = d_row_ptr;
    p.row_rank = d_row_rank;
    p.col_of_rank = d_col_of_rank;
    p.col_ptr = d_col_ptr;
    p.col_rows = d_col_rows;
    p.out_count = d_count;
    p.skipped = d_skipped;
    p.n_skipped = d_n_skipped;
    cudaMemset(p.hits, 0, (size_t)blocks * p.hits_stride * sizeof(u32));
    cudaMemset(p.bitmap, 0, (size_t)blocks * p.bitmap_stride * sizeof(u32));
    cudaMemset(d_n_skipped, 0, sizeof(i32));
    for (int attempt = 0; attempt < 2; ++attempt) {  // a second pass only if the output list was too small
        if ((e = cudaMalloc((void**)&p.out, (size_t)p.out_cap * sizeof(CandTriple))) != cudaSuccess) return fail("out", e);
        cudaMemset(d_count, 0, 2 * sizeof(u64));
        cudaMemset(d_n_skipped, 0, sizeof(i32));
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        const bool trace = std::getenv("CBM_B200_BUILD_TRACE") != nullptr;
        if (trace) {
            cudaEventCreate(&e0);
            cudaEventCreate(&e1);
            cudaEventRecord(e0);
        }
        candidate_kernel<<<blocks, kThreads>>>(p);
        if ((e = cudaGetLastError()) != cudaSuccess) return fail("launch", e);
        if (trace) cudaEventRecord(e1);
        if ((e = cudaDeviceSynchronize()) != cudaSuccess) return fail("kernel", e);
        if (trace) {
            float ms = 0.f;
            cudaEventElapsedTime(&ms, e0, e1);
            std::fprintf(stderr, "[cbm build] candidate kernel %.3f ms\n", ms);
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
        }
        u64 h_count[2] = {0, 0};
        cudaMemcpy(h_count, d_count, sizeof(h_count), cudaMemcpyDeviceToHost);
        if ((int64_t)h_count[0] <= p.out_cap) {
            out.resize((size_t)h_count[0]);
            if (h_count[0])
                cudaMemcpy(out.data(), p.out, (size_t)h_count[0] * sizeof(CandTriple), cudaMemcpyDeviceToHost);
            i32 ns = 0;
            cudaMemcpy(&ns, d_n_skipped, sizeof(ns), cudaMemcpyDeviceToHost);
            left_to_host.resize((size_t)ns);
            if (ns) cudaMemcpy(left_to_host.data(), d_skipped, (size_t)ns * sizeof(i32), cudaMemcpyDeviceToHost);
            cleanup();
            return 0;
        }
        cudaFree(p.out);
        p.out = nullptr;
        p.out_cap = (int64_t)h_count[0] + 1024;  // the kernel counted every survivor: now it fits
    }
    err = "gpu_candidates: output list overflowed twice";
    cleanup();
    return 1;
}

}  // namespace cbm
