// CUDA engine (sm_100a) for the CBM product: plans, kernels and the compute half of the C ABI.
//
// What the reference does in two steps per call — an MKL sparse product dst = deltas * rhs
// (cbm/cbm_extensions.cpp:694-704) followed by a depth-first walk that adds every finished parent
// row into its children (cbm/cbm_extensions.cpp:1166-1218; normalized form :1285-1373) — is done
// here by ONE kernel.  Rows are issued to warps in a topological order of the tree.  A warp
//   1. gathers the signed rows of X named by its row's delta entries into registers,
//   2. waits (bounded) until its parent's finished row is published, reads it from L2,
//   3. applies the row scale, stores the finished row once, and publishes it.
// Step 1 does not depend on the parent, so the wait in step 2 is normally already satisfied.
// The dense operand is processed in column slabs so that one slab of X stays resident in the
// 126 MB L2 while every row gathers from it.
//
// Forward progress: work items are claimed in increasing order from one counter, and an item only
// ever waits for an item with a smaller index.  Whoever holds that smaller item is already running
// and, by induction, never blocked on anything unclaimed, so the kernel cannot deadlock however
// many thread blocks are resident.  Every wait is bounded all the same: when the bound runs out
// the warp raises the plan's status word and all warps drain.

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "cbm_b200.h"
#include "cbm_common.h"

namespace cbm {
std::string& last_error_slot() {
    static thread_local std::string slot;
    return slot;
}
}  // namespace cbm

extern "C" const char* cbm_b200_last_error(void) { return cbm::last_error_slot().c_str(); }
extern "C" const char* cbm_b200_version(void) { return "cbm_b200 0.1 sm_100a"; }

namespace {

using i32 = int32_t;
using i64 = int64_t;
using u64 = unsigned long long;

#define CBM_CUDA(call)                                                                      \
    do {                                                                                    \
        cudaError_t e__ = (call);                                                           \
        if (e__ != cudaSuccess)                                                             \
            return cbm::fail(CBM_B200_ERR_CUDA, std::string(#call) + ": " +                 \
                                                    cudaGetErrorString(e__));               \
    } while (0)

// One work item of the schedule, in processing order.  32 bytes, read as two 16-byte loads.
// A row with many delta entries is cut into segments: all but the last become PARTIAL items that
// leave their share of the gather in a scratch slot; the last item of the row (placed directly
// after them) adds those slots to its own share and finishes the row.
struct __align__(16) RowDesc {
    i32 out_row;      // row of y this item produces (local to the shard); scratch slot if PARTIAL
    i32 parent_row;   // row of y holding the parent's finished row, -1 under the virtual root
    i32 parent_pos;   // parent's position in processing order (index of its ready flag)
    i32 flags;        // UNIT_* bits; bits 8.. = number of PARTIAL items directly before this one
    i32 beg, end;     // delta entries of the item in the plan's col/val arrays
    float scale;      // s_v  = D^-1/2 of this row (1 when the plan has no multiplier)
    float inv_parent; // 1/s_u of the parent (1 when none)
};
enum : int { UNIT_PUBLISH = 1, UNIT_PARTIAL = 2, UNIT_NPART_SHIFT = 8 };

enum Mode : int { MODE_FUSED = 0, MODE_DELTA_ONLY = 1, MODE_UPDATE_ONLY = 2 };

struct KParams {
    const RowDesc* desc;
    const i32* col;
    const float* val;
    const float* x;
    float* y;
    i64 ldx, ldy;
    i32 f;
    i32 slab_w;     // columns per slab
    i32 n_items;    // work items per slab (rows + extra segments of long rows)
    i64 n_units;    // n_items * n_slabs
    float* scratch; // n_slabs * n_slots * slab_w floats: partial sums of long rows
    i32 n_slots;
    u64* counter;   // [0] next chunk to claim, [1] warps that have left; both 0 between launches
    u64 n_warps;    // warps in this launch
    i32* flags;     // n_slabs * n_items ready flags holding the epoch of the launch that set them
    i32 epoch;
    i32* status;    // 0 ok; non-zero: a wait gave up
    i32 mode;
    i32 use_scale;
    u64 wait_ns;
};

__device__ __forceinline__ i32 ld_acquire(const i32* p) {
    i32 v;
    asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release(i32* p, i32 v) {
    asm volatile("st.release.gpu.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ i32 ld_relaxed(const i32* p) {
    i32 v;
    asm volatile("ld.relaxed.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ u64 global_ns() {
    u64 t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait for `*flag == epoch`.  All lanes of the warp call it together.
__device__ __forceinline__ bool wait_ready(const i32* flag, i32 epoch, i32* status, u64 wait_ns) {
    if (ld_acquire(flag) == epoch) return true;
    const u64 t0 = global_ns();
    unsigned spins = 0;
    for (;;) {
        if (ld_acquire(flag) == epoch) return true;
        ++spins;
        if ((spins & 31u) == 0) {
            if (ld_relaxed(status) != 0) return false;  // someone else gave up: drain
            if (global_ns() - t0 > wait_ns) {
                atomicExch(status, CBM_B200_ERR_TIMEOUT);
                return false;
            }
        }
        __nanosleep(spins < 16 ? 20 : 200);
    }
}

template <bool V4>
struct Vec;
template <>
struct Vec<true> {
    using T = float4;
    static constexpr int E = 4;
    static __device__ __forceinline__ T zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
    static __device__ __forceinline__ T ld_ro(const float* p) { return __ldg((const float4*)p); }
    // Read-only fetch that is skipped (giving zeros) when `on` is false.  Written as volatile asm
    // so that a batch of fetches stays a batch: the compiler may not sink one below its use.
    static __device__ __forceinline__ T ld_ro_if(const float* p, bool on) {
        T v;
        asm volatile(
            "{\n\t.reg .pred q;\n\tsetp.ne.s32 q, %5, 0;\n\t"
            "mov.f32 %0, 0f00000000;\n\tmov.f32 %1, 0f00000000;\n\t"
            "mov.f32 %2, 0f00000000;\n\tmov.f32 %3, 0f00000000;\n\t"
            "@q ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];\n\t}"
            : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
            : "l"(p), "r"((int)on));
        return v;
    }
    static __device__ __forceinline__ T ld_l2(const float* p) { return __ldcg((const float4*)p); }
    static __device__ __forceinline__ void st(float* p, T v) { *(float4*)p = v; }
    static __device__ __forceinline__ T fma(float w, T a, T c) {
        c.x = fmaf(w, a.x, c.x);
        c.y = fmaf(w, a.y, c.y);
        c.z = fmaf(w, a.z, c.z);
        c.w = fmaf(w, a.w, c.w);
        return c;
    }
    static __device__ __forceinline__ T mul(float w, T a) {
        a.x *= w;
        a.y *= w;
        a.z *= w;
        a.w *= w;
        return a;
    }
};
template <>
struct Vec<false> {
    using T = float;
    static constexpr int E = 1;
    static __device__ __forceinline__ T zero() { return 0.f; }
    static __device__ __forceinline__ T ld_ro(const float* p) { return __ldg(p); }
    static __device__ __forceinline__ T ld_ro_if(const float* p, bool on) {
        T v;
        asm volatile(
            "{\n\t.reg .pred q;\n\tsetp.ne.s32 q, %2, 0;\n\tmov.f32 %0, 0f00000000;\n\t"
            "@q ld.global.nc.f32 %0, [%1];\n\t}"
            : "=f"(v)
            : "l"(p), "r"((int)on));
        return v;
    }
    static __device__ __forceinline__ T ld_l2(const float* p) { return __ldcg(p); }
    static __device__ __forceinline__ void st(float* p, T v) { *p = v; }
    static __device__ __forceinline__ T fma(float w, T a, T c) { return fmaf(w, a, c); }
    static __device__ __forceinline__ T mul(float w, T a) { return w * a; }
};

// A warp signs off; the last one out rewinds both counters for the next launch.  This holds on
// the drain path after a failed wait too, so a plan stays usable after a timeout.
__device__ __forceinline__ void leave(const KParams& p, int lane) {
    if (lane == 0) {
        if (atomicAdd(p.counter + 1, 1ULL) == p.n_warps - 1) {
            p.counter[0] = 0;
            p.counter[1] = 0;
            __threadfence();
        }
    }
}

// acc[v] += sum over entries [beg,end) of val * X[col, slab columns of this lane].
// The 32 lanes fetch 32 (col, val) pairs at once and pass them round by shuffle.  Row fetches are
// issued UNROLL at a time so that several independent loads per lane are in flight; the weights
// are picked up after the fetches have been issued.
template <int NV, bool V4, int UNROLL>
__device__ __forceinline__ void gather_row(const i32* __restrict__ col,
                                           const float* __restrict__ val, i32 beg, i32 end,
                                           const float* __restrict__ xs, i64 ldx,
                                           const bool (&ok)[NV], typename Vec<V4>::T (&acc)[NV],
                                           int lane) {
    using V = Vec<V4>;
    using T = typename V::T;
    constexpr int STEP = 32 * V::E;
    for (i32 b = beg; b < end; b += 32) {
        const i32 n_here = min(32, end - b);
        i32 mc = 0;
        float mw = 0.f;
        if (lane < n_here) {
            mc = __ldg(col + b + lane);
            mw = __ldg(val + b + lane);
        }
        i32 j = 0;
        for (; j + UNROLL <= n_here; j += UNROLL) {
            T t[UNROLL][NV];
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                const i32 c = __shfl_sync(0xffffffffu, mc, j + k);
                const float* r = xs + (i64)c * ldx;
#pragma unroll
                for (int v = 0; v < NV; ++v) t[k][v] = V::ld_ro_if(r + v * STEP, ok[v]);
            }
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                const float w = __shfl_sync(0xffffffffu, mw, j + k);
#pragma unroll
                for (int v = 0; v < NV; ++v) acc[v] = V::fma(w, t[k][v], acc[v]);
            }
        }
        for (; j < n_here; ++j) {
            const i32 c = __shfl_sync(0xffffffffu, mc, j);
            const float w = __shfl_sync(0xffffffffu, mw, j);
            const float* r = xs + (i64)c * ldx;
#pragma unroll
            for (int v = 0; v < NV; ++v)
                if (ok[v]) acc[v] = V::fma(w, V::ld_ro(r + v * STEP), acc[v]);
        }
    }
}

// The fused product kernel.  One warp per (row segment, column slab) item; NV vectors per lane.
// UNROLL = row fetches in flight per lane, MINB = thread blocks the register budget must allow
// per SM.
template <int NV, bool V4, int UNROLL, int MINB>
__global__ void __launch_bounds__(256, MINB) cbm_rows_kernel(const KParams p) {
    using V = Vec<V4>;
    using T = typename V::T;
    constexpr int STEP = 32 * V::E;
    const int lane = threadIdx.x & 31;
    for (;;) {
        u64 t = 0;
        if (lane == 0) t = atomicAdd(p.counter, 1ULL);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (t >= (u64)p.n_units) {
            leave(p, lane);
            return;
        }
        // One item per claim.  Handing a warp several consecutive items makes it sit on an item
        // that waits for a neighbour while the items behind it (which others wait for) starve.
        {
            const unsigned u = (unsigned)t;  // the host refuses launches of 2^31 items or more
            const i32 slab = (i32)(u / (unsigned)p.n_items);
            const i32 pos = (i32)(u - (unsigned)slab * (unsigned)p.n_items);
            const int4 da = __ldg((const int4*)(p.desc + pos));
            const int4 db = __ldg((const int4*)(p.desc + pos) + 1);
            const i32 out_row = da.x, parent_row = da.y, parent_pos = da.z, flags = da.w;
            const i32 beg = db.x, end = db.y;
            const float scale = __int_as_float(db.z), inv_parent = __int_as_float(db.w);
            const bool partial = (flags & UNIT_PARTIAL) != 0;
            if (partial && p.mode == MODE_UPDATE_ONLY) continue;
            const i32 c0 = slab * p.slab_w;
            const i32 wcols = min(p.slab_w, p.f - c0);
            const i32 lane_col = c0 + lane * V::E;
            bool ok[NV];
#pragma unroll
            for (int v = 0; v < NV; ++v) ok[v] = (lane * V::E + v * STEP) < wcols;
            i32* my_flag = p.flags + (i64)slab * p.n_items + pos;
            T acc[NV];
            float* yrow = p.y + (i64)out_row * p.ldy + lane_col;
            if (p.mode == MODE_UPDATE_ONLY) {
#pragma unroll
                for (int v = 0; v < NV; ++v) acc[v] = ok[v] ? V::ld_l2(yrow + v * STEP) : V::zero();
            } else {
#pragma unroll
                for (int v = 0; v < NV; ++v) acc[v] = V::zero();
                gather_row<NV, V4, UNROLL>(p.col, p.val, beg, end, p.x + lane_col, p.ldx, ok, acc, lane);
            }
            if (partial) {
                float* slot = p.scratch + ((i64)slab * p.n_slots + out_row) * p.slab_w + lane * V::E;
#pragma unroll
                for (int v = 0; v < NV; ++v)
                    if (ok[v]) V::st(slot + v * STEP, acc[v]);
                __threadfence();
                __syncwarp();
                if (lane == 0) st_release(my_flag, p.epoch);
                continue;
            }
            const i32 n_part = flags >> UNIT_NPART_SHIFT;
            if (n_part > 0 && p.mode != MODE_UPDATE_ONLY) {
                const i32 last_slot = __ldg(&p.desc[pos - 1].out_row);
                for (i32 k = 0; k < n_part; ++k) {
                    if (!wait_ready(my_flag - n_part + k, p.epoch, p.status, p.wait_ns)) {
                        leave(p, lane);
                        return;
                    }
                    const float* slot = p.scratch +
                                        ((i64)slab * p.n_slots + (last_slot - (n_part - 1) + k)) * p.slab_w +
                                        lane * V::E;
#pragma unroll
                    for (int v = 0; v < NV; ++v)
                        if (ok[v]) acc[v] = V::fma(1.0f, V::ld_l2(slot + v * STEP), acc[v]);
                }
            }
            if (p.mode != MODE_DELTA_ONLY) {
                if (parent_row >= 0) {
                    if (!wait_ready(p.flags + (i64)slab * p.n_items + parent_pos, p.epoch, p.status,
                                    p.wait_ns)) {
                        leave(p, lane);
                        return;
                    }
                    const float* prow = p.y + (i64)parent_row * p.ldy + lane_col;
                    const float ip = p.use_scale ? inv_parent : 1.0f;
#pragma unroll
                    for (int v = 0; v < NV; ++v)
                        if (ok[v]) acc[v] = V::fma(ip, V::ld_l2(prow + v * STEP), acc[v]);
                }
                if (p.use_scale) {
#pragma unroll
                    for (int v = 0; v < NV; ++v) acc[v] = V::mul(scale, acc[v]);
                }
            }
#pragma unroll
            for (int v = 0; v < NV; ++v)
                if (ok[v]) V::st(yrow + v * STEP, acc[v]);
            if ((flags & UNIT_PUBLISH) && p.mode != MODE_DELTA_ONLY) {
                __threadfence();
                __syncwarp();
                if (lane == 0) st_release(my_flag, p.epoch);
            }
        }
    }
}
// Plain CSR product (no tree): rows in natural order, one warp per (row, slab), grid-stride.
template <int NV, bool V4>
__global__ void __launch_bounds__(256)
    csr_rows_kernel(i32 n_rows, const i32* __restrict__ row_b, const i32* __restrict__ row_e,
                    const i32* __restrict__ col, const float* __restrict__ val,
                    const float* __restrict__ x, i64 ldx, float* __restrict__ y, i64 ldy, i32 f,
                    i32 slab_w, i64 n_units) {
    using V = Vec<V4>;
    using T = typename V::T;
    constexpr int STEP = 32 * V::E;
    const int lane = threadIdx.x & 31;
    const i64 warp = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const i64 n_warps = ((i64)gridDim.x * blockDim.x) >> 5;
    for (i64 u = warp; u < n_units; u += n_warps) {
        const i32 slab = (i32)(u / n_rows);
        const i32 row = (i32)(u - (i64)slab * n_rows);
        const i32 c0 = slab * slab_w;
        const i32 wcols = min(slab_w, f - c0);
        const i32 lane_col = c0 + lane * V::E;
        bool ok[NV];
        T acc[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            ok[v] = (lane * V::E + v * STEP) < wcols;
            acc[v] = V::zero();
        }
        gather_row<NV, V4, (NV >= 4 ? 4 : 8)>(col, val, __ldg(row_b + row), __ldg(row_e + row), x + lane_col, ldx, ok,
                           acc, lane);
        float* yrow = y + (i64)row * ldy + lane_col;
#pragma unroll
        for (int v = 0; v < NV; ++v)
            if (ok[v]) V::st(yrow + v * STEP, acc[v]);
    }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Picks the widest vector form the operands allow and the slab width it covers.
struct Shape {
    bool v4;
    int nv;
    i32 slab_w;
    i32 n_slabs;
};
Shape pick_shape(i32 f, i32 want_slab, bool can_v4) {
    Shape s{};
    s.v4 = can_v4;
    const i32 lane_w = s.v4 ? 128 : 32;  // columns covered by one vector per lane
    i32 slab = want_slab > 0 ? want_slab : (s.v4 ? 256 : 64);
    slab = std::max(lane_w, (slab / lane_w) * lane_w);
    slab = std::min(slab, lane_w * 4);
    const i32 f_up = ((f + lane_w - 1) / lane_w) * lane_w;
    slab = std::min(slab, f_up);
    s.nv = slab / lane_w;
    if (s.nv == 3) {
        s.nv = 2;
        slab = 2 * lane_w;
    }
    s.slab_w = slab;
    s.n_slabs = (f + slab - 1) / slab;
    return s;
}

}  // namespace

// ------------------------------------------------------------------------------------------
struct cbm_b200_plan {
    int device = 0;
    i32 n = 0;
    i32 n_labels = 0;  // rows of the dense right-hand side
    i32 n_out = 0;     // rows of the output shard (owned label range)
    i32 n_rows = 0;    // rows actually computed
    i32 n_items = 0;   // work items per slab (rows + extra segments of long rows)
    i32 n_slots = 0;   // scratch slots per slab
    float* d_scratch = nullptr;
    i64 scratch_cap = 0;
    i64 n_delta = 0;
    i32 n_root_children = 0;
    i32 depth = 0;
    bool normalized = false;
    RowDesc* d_desc = nullptr;
    i32* d_col = nullptr;
    float* d_val = nullptr;
    i32* d_flags = nullptr;
    i64 flags_cap = 0;
    u64* d_counter = nullptr;
    i32* d_status = nullptr;
    i32 epoch = 0;
    i32 slab_width = 0;
    i32 n_blocks = 0;
    i32 sm_count = 148;
    i64 device_bytes = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    std::vector<cudaEvent_t> events;
    i32 host_chunk = 0;
    float* stage_x = nullptr;
    float* stage_y = nullptr;
    i64 stage_x_cap = 0, stage_y_cap = 0;
};

namespace {

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

template <class T>
int upload(T** dst, const std::vector<T>& src, i64& bytes) {
    *dst = nullptr;
    const size_t sz = std::max<size_t>(src.size(), 1) * sizeof(T);
    CBM_CUDA(cudaMalloc((void**)dst, sz));
    bytes += (i64)sz;
    if (!src.empty())
        CBM_CUDA(cudaMemcpy(*dst, src.data(), src.size() * sizeof(T), cudaMemcpyHostToDevice));
    return CBM_B200_OK;
}

}  // namespace

extern "C" void cbm_b200_plan_destroy(cbm_b200_plan* p) {
    if (!p) return;
    DeviceGuard g(p->device);
    cudaFree(p->d_desc);
    cudaFree(p->d_col);
    cudaFree(p->d_val);
    cudaFree(p->d_flags);
    cudaFree(p->d_scratch);
    cudaFree(p->d_counter);
    cudaFree(p->d_status);
    cudaFree(p->stage_x);
    cudaFree(p->stage_y);
    if (p->own_stream) cudaStreamDestroy(p->own_stream);
    if (p->copy_in) cudaStreamDestroy(p->copy_in);
    if (p->copy_out) cudaStreamDestroy(p->copy_out);
    for (cudaEvent_t e : p->events) cudaEventDestroy(e);
    delete p;
}

extern "C" int cbm_b200_plan_create(int32_t n, const int32_t* mst_row, const int32_t* mst_col,
                                    const int32_t* delta_crow, const int32_t* delta_col,
                                    const float* delta_val, const float* multiplier,
                                    const int32_t* perm, int32_t n_labels, int32_t own_begin,
                                    int32_t own_end, int32_t device, cbm_b200_plan** out) {
    if (!out) return cbm::fail(CBM_B200_ERR_ARG, "plan_create: out is NULL");
    *out = nullptr;
    if (n < 0 || !mst_row || !delta_crow || (n > 0 && !mst_col))
        return cbm::fail(CBM_B200_ERR_ARG, "plan_create: NULL tree or delta arrays");
    if (n_labels == 0) n_labels = n;
    if (n_labels < n || (!perm && n_labels != n))
        return cbm::fail(CBM_B200_ERR_ARG, "plan_create: n_labels must be >= n (== n without perm)");
    if (own_begin < 0 || own_end > n_labels || own_begin > own_end)
        return cbm::fail(CBM_B200_ERR_ARG, "plan_create: bad owned range");
    const i64 nd_all = delta_crow[n];
    if (nd_all > 0 && (!delta_col || !delta_val))
        return cbm::fail(CBM_B200_ERR_ARG, "plan_create: NULL delta col/val");

    // ---- validate the tree: every row exactly once, reachable from the virtual root ----
    if (mst_row[0] != 0 || mst_row[n + 1] != n)
        return cbm::fail(CBM_B200_ERR_FORMAT, "plan_create: mst_row must run from 0 to n");
    std::vector<i32> parent((size_t)n, -1);
    for (i32 u = 0; u <= n; ++u) {
        if (mst_row[u] > mst_row[u + 1])
            return cbm::fail(CBM_B200_ERR_FORMAT, "plan_create: mst_row not monotone");
        for (i32 k = mst_row[u]; k < mst_row[u + 1]; ++k) {
            const i32 v = mst_col[k];
            if (v < 0 || v >= n || parent[v] != -1 || v == u)
                return cbm::fail(CBM_B200_ERR_FORMAT,
                                 "plan_create: mst_col is not a tree over the rows");
            parent[v] = u;
        }
    }
    std::vector<i32> order;  // breadth-first from the virtual root
    order.reserve((size_t)n);
    std::vector<i32> level((size_t)n + 1, 0);
    {
        std::vector<i32> q;
        q.reserve((size_t)n + 1);
        q.push_back(n);
        for (size_t h = 0; h < q.size(); ++h) {
            const i32 u = q[h];
            for (i32 k = mst_row[u]; k < mst_row[u + 1]; ++k) {
                level[mst_col[k]] = level[u] + 1;
                q.push_back(mst_col[k]);
            }
        }
        if ((i32)q.size() != n + 1)
            return cbm::fail(CBM_B200_ERR_FORMAT, "plan_create: tree has a cycle or unreachable rows");
        order.assign(q.begin() + 1, q.end());
    }
    for (i32 v = 0; v < n; ++v) {
        if (delta_crow[v] > delta_crow[v + 1] || delta_crow[v] < 0)
            return cbm::fail(CBM_B200_ERR_FORMAT, "plan_create: delta_crow not monotone");
    }
    for (i64 k = 0; k < nd_all; ++k)
        if (delta_col[k] < 0 || delta_col[k] >= n)
            return cbm::fail(CBM_B200_ERR_FORMAT, "plan_create: delta column out of range");
    if (perm) {
        std::vector<char> seen((size_t)n_labels, 0);
        for (i32 v = 0; v < n; ++v) {
            if (perm[v] < 0 || perm[v] >= n_labels || seen[perm[v]])
                return cbm::fail(CBM_B200_ERR_ARG, "plan_create: perm labels not distinct / in range");
            seen[perm[v]] = 1;
        }
    }
    auto label = [&](i32 v) { return perm ? perm[v] : v; };
    auto owned = [&](i32 v) {
        const i32 l = label(v);
        return l >= own_begin && l < own_end;
    };

    // ---- schedule ----
    // Owned rows in breadth-first order, except that the children of the virtual root (which wait
    // for nobody) are issued longest first so that the heavy rows never form the tail.  Any order
    // in which a parent precedes its children is valid.
    std::vector<i32> sched;
    sched.reserve((size_t)(own_end - own_begin));
    for (i32 v : order)
        if (owned(v)) sched.push_back(v);
    {
        auto first_deep = std::stable_partition(sched.begin(), sched.end(),
                                                [&](i32 v) { return parent[v] == n; });
        std::stable_sort(sched.begin(), first_deep, [&](i32 a, i32 b) {
            return delta_crow[a + 1] - delta_crow[a] > delta_crow[b + 1] - delta_crow[b];
        });
    }
    const i32 SEG = 128;        // delta entries per work item of a long row
    const i32 SPLIT_OVER = 192; // rows longer than this are cut into segments
    std::vector<i32> pos_of((size_t)n, -1);
    std::vector<RowDesc> desc;
    desc.reserve(sched.size());
    std::vector<i32> pcol;
    std::vector<float> pval;
    pcol.reserve((size_t)nd_all);
    pval.reserve((size_t)nd_all);
    i32 depth = 0, n_root_children = 0, n_slots = 0;
    for (i32 v : sched) {
        const i32 u = parent[v];
        if (u != n && !owned(u))
            return cbm::fail(CBM_B200_ERR_ARG,
                             "plan_create: owned range cuts a subtree (parent of an owned row "
                             "is not owned)");
        const i32 first = (i32)pcol.size();
        for (i32 k = delta_crow[v]; k < delta_crow[v + 1]; ++k) {
            pcol.push_back(label(delta_col[k]));
            pval.push_back(delta_val[k]);
        }
        const i32 len = (i32)pcol.size() - first;
        i32 n_part = 0;
        i32 cursor = first;
        if (len > SPLIT_OVER) {
            const i32 n_seg = (len + SEG - 1) / SEG;
            n_part = n_seg - 1;
            for (i32 k = 0; k < n_part; ++k) {
                RowDesc q{};
                q.out_row = n_slots++;
                q.parent_row = -1;
                q.parent_pos = -1;
                q.flags = UNIT_PARTIAL | UNIT_PUBLISH;
                q.beg = cursor;
                q.end = cursor + SEG;
                q.scale = 1.0f;
                q.inv_parent = 1.0f;
                cursor += SEG;
                desc.push_back(q);
            }
        }
        RowDesc d{};
        d.out_row = label(v) - own_begin;
        d.parent_row = (u == n) ? -1 : label(u) - own_begin;
        d.parent_pos = (u == n) ? -1 : pos_of[u];
        d.flags = n_part << UNIT_NPART_SHIFT;
        d.beg = cursor;
        d.end = (i32)pcol.size();
        d.scale = multiplier ? multiplier[v] : 1.0f;
        d.inv_parent = (multiplier && u != n) ? 1.0f / multiplier[u] : 1.0f;
        pos_of[v] = (i32)desc.size();
        if (u != n) desc[pos_of[u]].flags |= UNIT_PUBLISH;
        else ++n_root_children;
        depth = std::max(depth, level[v]);
        desc.push_back(d);
    }
    const i32 n_rows_owned = (i32)sched.size();

    int n_dev = 0;
    CBM_CUDA(cudaGetDeviceCount(&n_dev));
    if (device < 0 || device >= n_dev)
        return cbm::fail(CBM_B200_ERR_ARG, "plan_create: no such CUDA device");
    DeviceGuard guard(device);
    if (!guard.ok) return cbm::fail(CBM_B200_ERR_CUDA, "plan_create: cudaSetDevice failed");

    cbm_b200_plan* p = new (std::nothrow) cbm_b200_plan();
    if (!p) return cbm::fail(CBM_B200_ERR_ALLOC, "plan_create: out of host memory");
    p->device = device;
    p->n = n;
    p->n_labels = n_labels;
    p->n_out = own_end - own_begin;
    p->n_rows = n_rows_owned;
    p->n_items = (i32)desc.size();
    p->n_slots = n_slots;
    p->n_delta = (i64)pcol.size();
    p->n_root_children = n_root_children;
    p->depth = depth;
    p->normalized = multiplier != nullptr;
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) p->sm_count = prop.multiProcessorCount;
    int rc = upload(&p->d_desc, desc, p->device_bytes);
    if (rc == CBM_B200_OK) rc = upload(&p->d_col, pcol, p->device_bytes);
    if (rc == CBM_B200_OK) rc = upload(&p->d_val, pval, p->device_bytes);
    if (rc == CBM_B200_OK) {
        cudaError_t e = cudaMalloc((void**)&p->d_counter, 2 * sizeof(u64));
        if (e == cudaSuccess) e = cudaMemset(p->d_counter, 0, 2 * sizeof(u64));
        if (e == cudaSuccess) e = cudaMalloc((void**)&p->d_status, sizeof(i32));
        if (e == cudaSuccess) e = cudaMemset(p->d_status, 0, sizeof(i32));
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&p->own_stream, cudaStreamNonBlocking);
        if (e != cudaSuccess)
            rc = cbm::fail(CBM_B200_ERR_CUDA, std::string("plan_create: ") + cudaGetErrorString(e));
        p->device_bytes += 16;
    }
    if (rc != CBM_B200_OK) {
        const std::string keep = cbm::last_error_slot();
        cbm_b200_plan_destroy(p);
        cbm::last_error_slot() = keep;
        return rc;
    }
    *out = p;
    return CBM_B200_OK;
}

extern "C" int cbm_b200_plan_info(const cbm_b200_plan* p, int32_t* n_rows, int64_t* n_delta,
                                  int32_t* n_root_children, int32_t* depth,
                                  int64_t* device_bytes) {
    if (!p) return cbm::fail(CBM_B200_ERR_ARG, "plan_info: NULL plan");
    if (n_rows) *n_rows = p->n_rows;
    if (n_delta) *n_delta = p->n_delta;
    if (n_root_children) *n_root_children = p->n_root_children;
    if (depth) *depth = p->depth;
    if (device_bytes) *device_bytes = p->device_bytes;
    return CBM_B200_OK;
}

extern "C" int cbm_b200_plan_tune(cbm_b200_plan* p, int32_t slab_width, int32_t n_blocks,
                                  int32_t host_chunk) {
    if (!p) return cbm::fail(CBM_B200_ERR_ARG, "plan_tune: NULL plan");
    if (slab_width < 0 || n_blocks < 0 || host_chunk < 0)
        return cbm::fail(CBM_B200_ERR_ARG, "plan_tune: negative knob");
    if (host_chunk % 4 != 0) return cbm::fail(CBM_B200_ERR_ARG, "plan_tune: host_chunk must be a multiple of 4");
    p->slab_width = slab_width;
    p->n_blocks = n_blocks;
    p->host_chunk = host_chunk;
    return CBM_B200_OK;
}

extern "C" int cbm_b200_plan_status(cbm_b200_plan* p, void* stream) {
    if (!p) return cbm::fail(CBM_B200_ERR_ARG, "plan_status: NULL plan");
    DeviceGuard g(p->device);
    CBM_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    i32 st = 0;
    CBM_CUDA(cudaMemcpy(&st, p->d_status, sizeof(st), cudaMemcpyDeviceToHost));
    if (st != 0) {
        CBM_CUDA(cudaMemset(p->d_status, 0, sizeof(i32)));
        return cbm::fail(CBM_B200_ERR_TIMEOUT,
                         "a bounded wait for a parent row ran out; the last product is invalid");
    }
    return CBM_B200_OK;
}

namespace {

template <int NV, bool V4>
int launch_rows(const KParams& kp, int blocks, cudaStream_t s) {
    // Unroll depth and resident blocks per SM were chosen by measurement on B200: forms that
    // spill registers lose more than extra resident warps gain.
    cbm_rows_kernel<NV, V4, (NV == 1 ? 8 : 4), (NV == 1 ? 4 : (NV == 2 ? 3 : 2))><<<blocks, 256, 0, s>>>(kp);
    CBM_CUDA(cudaGetLastError());
    return CBM_B200_OK;
}

int check_dense(const char* who, const void* x, i64 ldx, const void* y, i64 ldy, i32 f) {
    if (f <= 0) return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": f must be positive");
    if (!y || ldy < f) return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": bad y / ldy");
    if (x && ldx < f) return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": ldx < f");
    if (ldx > INT32_MAX || ldy > INT32_MAX)
        return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": leading dimension exceeds 2^31-1");
    if (x && x == y) return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": x and y alias");
    return CBM_B200_OK;
}

int run_plan(cbm_b200_plan* p, const char* who, const float* x, i64 ldx, float* y, i64 ldy, i32 f,
             int mode, bool use_scale, cudaStream_t s) {
    if (!p) return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": NULL plan");
    int rc = check_dense(who, x, ldx, y, ldy, f);
    if (rc) return rc;
    if (mode != MODE_UPDATE_ONLY && !x)
        return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": x is NULL");
    if (use_scale && !p->normalized)
        return cbm::fail(CBM_B200_ERR_ARG,
                         std::string(who) + ": plan was created without a multiplier");
    if (p->n_rows == 0) return CBM_B200_OK;
    DeviceGuard g(p->device);

    const bool can_v4 = (f % 4 == 0) && (ldy % 4 == 0) && aligned16(y) &&
                        (mode == MODE_UPDATE_ONLY || ((ldx % 4 == 0) && aligned16(x)));
    const Shape sh = pick_shape(f, p->slab_width, can_v4);

    const i64 need_flags = (i64)sh.n_slabs * p->n_items;
    if (need_flags >= (i64)1 << 31)
        return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": rows x column slabs exceeds 2^31 work items");
    if (need_flags > p->flags_cap) {
        // Growing the flag array: the old one may still be read by a launch in flight.
        CBM_CUDA(cudaStreamSynchronize(s));
        cudaFree(p->d_flags);
        p->d_flags = nullptr;
        p->device_bytes -= p->flags_cap * (i64)sizeof(i32);
        p->flags_cap = 0;
        CBM_CUDA(cudaMalloc((void**)&p->d_flags, (size_t)need_flags * sizeof(i32)));
        CBM_CUDA(cudaMemset(p->d_flags, 0, (size_t)need_flags * sizeof(i32)));
        p->flags_cap = need_flags;
        p->device_bytes += need_flags * (i64)sizeof(i32);
    }
    const i64 need_scratch = (i64)sh.n_slabs * p->n_slots * sh.slab_w;
    if (need_scratch > p->scratch_cap) {
        CBM_CUDA(cudaStreamSynchronize(s));
        cudaFree(p->d_scratch);
        p->d_scratch = nullptr;
        p->device_bytes -= p->scratch_cap * (i64)sizeof(float);
        p->scratch_cap = 0;
        CBM_CUDA(cudaMalloc((void**)&p->d_scratch, (size_t)need_scratch * sizeof(float)));
        p->scratch_cap = need_scratch;
        p->device_bytes += need_scratch * (i64)sizeof(float);
    }
    if (p->epoch == INT32_MAX) {  // epochs exhausted: start over on clean flags
        CBM_CUDA(cudaMemsetAsync(p->d_flags, 0, (size_t)p->flags_cap * sizeof(i32), s));
        p->epoch = 0;
    }

    KParams kp{};
    kp.desc = p->d_desc;
    kp.col = p->d_col;
    kp.val = p->d_val;
    kp.x = x;
    kp.y = y;
    kp.ldx = ldx;
    kp.ldy = ldy;
    kp.f = f;
    kp.slab_w = sh.slab_w;
    kp.n_items = p->n_items;
    kp.scratch = p->d_scratch;
    kp.n_slots = p->n_slots;
    kp.n_units = need_flags;
    kp.counter = p->d_counter;
    kp.flags = p->d_flags;
    kp.epoch = ++p->epoch;
    kp.status = p->d_status;
    kp.mode = mode;
    kp.use_scale = use_scale ? 1 : 0;
    kp.wait_ns = 2000000000ULL;

    int blocks = p->n_blocks > 0 ? p->n_blocks : p->sm_count * 8;
    const i64 max_useful = (kp.n_units + 7) / 8;
    blocks = (int)std::max<i64>(1, std::min<i64>(blocks, max_useful));
    kp.n_warps = (u64)blocks * 8;

    if (sh.v4) {
        if (sh.nv == 1) return launch_rows<1, true>(kp, blocks, s);
        if (sh.nv == 2) return launch_rows<2, true>(kp, blocks, s);
        return launch_rows<4, true>(kp, blocks, s);
    }
    if (sh.nv == 1) return launch_rows<1, false>(kp, blocks, s);
    if (sh.nv == 2) return launch_rows<2, false>(kp, blocks, s);
    return launch_rows<4, false>(kp, blocks, s);
}

}  // namespace

extern "C" int cbm_b200_spmm_update(cbm_b200_plan* p, const float* x, int64_t ldx, float* y,
                                    int64_t ldy, int32_t f, void* stream) {
    return run_plan(p, "spmm_update", x, ldx, y, ldy, f, MODE_FUSED, false, (cudaStream_t)stream);
}
extern "C" int cbm_b200_fused_spmm_update(cbm_b200_plan* p, const float* x, int64_t ldx, float* y,
                                          int64_t ldy, int32_t f, void* stream) {
    return run_plan(p, "fused_spmm_update", x, ldx, y, ldy, f, MODE_FUSED, true,
                    (cudaStream_t)stream);
}
extern "C" int cbm_b200_update(cbm_b200_plan* p, float* y, int64_t ldy, int32_t f, void* stream) {
    return run_plan(p, "update", nullptr, 0, y, ldy, f, MODE_UPDATE_ONLY, false,
                    (cudaStream_t)stream);
}
extern "C" int cbm_b200_fused_update(cbm_b200_plan* p, float* y, int64_t ldy, int32_t f,
                                     void* stream) {
    return run_plan(p, "fused_update", nullptr, 0, y, ldy, f, MODE_UPDATE_ONLY, true,
                    (cudaStream_t)stream);
}
extern "C" int cbm_b200_delta_spmm(cbm_b200_plan* p, const float* x, int64_t ldx, float* y,
                                   int64_t ldy, int32_t f, void* stream) {
    return run_plan(p, "delta_spmm", x, ldx, y, ldy, f, MODE_DELTA_ONLY, false,
                    (cudaStream_t)stream);
}

extern "C" int cbm_b200_csr_spmm(int32_t n_rows, const int32_t* row_b, const int32_t* row_e,
                                 const int32_t* col, const float* val, const float* x,
                                 int64_t ldx, float* y, int64_t ldy, int32_t f, void* stream) {
    if (n_rows < 0 || (n_rows > 0 && (!row_b || !row_e)))
        return cbm::fail(CBM_B200_ERR_ARG, "csr_spmm: bad row arrays");
    int rc = check_dense("csr_spmm", x, ldx, y, ldy, f);
    if (rc) return rc;
    if (!x) return cbm::fail(CBM_B200_ERR_ARG, "csr_spmm: x is NULL");
    if (n_rows == 0) return CBM_B200_OK;
    const bool can_v4 = (f % 4 == 0) && (ldy % 4 == 0) && (ldx % 4 == 0) && aligned16(y) && aligned16(x);
    const Shape sh = pick_shape(f, 0, can_v4);
    const i64 n_units = (i64)sh.n_slabs * n_rows;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess)
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int blocks = (int)std::max<i64>(1, std::min<i64>((i64)sms * 8, (n_units + 7) / 8));
    cudaStream_t s = (cudaStream_t)stream;
#define CBM_CSR_LAUNCH(NV, V4)                                                                    \
    csr_rows_kernel<NV, V4><<<blocks, 256, 0, s>>>(n_rows, row_b, row_e, col, val, x, ldx, y, ldy, \
                                                   f, sh.slab_w, n_units)
    if (sh.v4) {
        if (sh.nv == 1) CBM_CSR_LAUNCH(1, true);
        else if (sh.nv == 2) CBM_CSR_LAUNCH(2, true);
        else CBM_CSR_LAUNCH(4, true);
    } else {
        if (sh.nv == 1) CBM_CSR_LAUNCH(1, false);
        else if (sh.nv == 2) CBM_CSR_LAUNCH(2, false);
        else CBM_CSR_LAUNCH(4, false);
    }
#undef CBM_CSR_LAUNCH
    CBM_CUDA(cudaGetLastError());
    return CBM_B200_OK;
}

extern "C" int cbm_b200_spmm_update_host(cbm_b200_plan* p, const float* x, float* y, int32_t f,
                                         int32_t normalized) {
    if (!p) return cbm::fail(CBM_B200_ERR_ARG, "spmm_update_host: NULL plan");
    if (!x || !y || f <= 0) return cbm::fail(CBM_B200_ERR_ARG, "spmm_update_host: bad x / y / f");
    DeviceGuard g(p->device);
    // leading dimension rounded up to 4 floats so the 128-bit path applies to any f % 4 == 0
    const i64 xb = (i64)p->n_labels * f, yb = (i64)p->n_out * f;
    if (xb > p->stage_x_cap) {
        cudaFree(p->stage_x);
        p->stage_x = nullptr;
        p->stage_x_cap = 0;
        CBM_CUDA(cudaMalloc((void**)&p->stage_x, (size_t)xb * sizeof(float)));
        p->stage_x_cap = xb;
    }
    if (yb > p->stage_y_cap) {
        cudaFree(p->stage_y);
        p->stage_y = nullptr;
        p->stage_y_cap = 0;
        CBM_CUDA(cudaMalloc((void**)&p->stage_y, (size_t)std::max<i64>(yb, 1) * sizeof(float)));
        // padding rows of a shard are never written by the kernel: give them a defined value
        CBM_CUDA(cudaMemset(p->stage_y, 0, (size_t)std::max<i64>(yb, 1) * sizeof(float)));
        p->stage_y_cap = yb;
    }
    // Pipeline over column chunks: while chunk k is multiplied, chunk k+1 of x is on its way in
    // and chunk k-1 of y on its way out (PCIe is full duplex), so the call costs about one
    // transfer of x plus the last chunk's product and transfer instead of x + product + y.
    const i32 chunk = p->host_chunk > 0 ? p->host_chunk : 128;
    const i32 n_chunks = (f + chunk - 1) / chunk;
    if (!p->copy_in) CBM_CUDA(cudaStreamCreateWithFlags(&p->copy_in, cudaStreamNonBlocking));
    if (!p->copy_out) CBM_CUDA(cudaStreamCreateWithFlags(&p->copy_out, cudaStreamNonBlocking));
    while ((i32)p->events.size() < 2 * n_chunks) {
        cudaEvent_t e;
        CBM_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        p->events.push_back(e);
    }
    cudaStream_t s = p->own_stream;
    const size_t pitch = (size_t)f * sizeof(float);
    for (i32 k = 0; k < n_chunks; ++k) {
        const i32 c0 = k * chunk;
        const i32 w = std::min(chunk, f - c0);
        CBM_CUDA(cudaMemcpy2DAsync(p->stage_x + c0, pitch, x + c0, pitch, (size_t)w * sizeof(float),
                                   (size_t)p->n_labels, cudaMemcpyHostToDevice, p->copy_in));
        CBM_CUDA(cudaEventRecord(p->events[2 * k], p->copy_in));
        CBM_CUDA(cudaStreamWaitEvent(s, p->events[2 * k], 0));
        int rc = run_plan(p, "spmm_update_host", p->stage_x + c0, f, p->stage_y + c0, f, w, MODE_FUSED,
                          normalized != 0, s);
        if (rc) return rc;
        CBM_CUDA(cudaEventRecord(p->events[2 * k + 1], s));
        CBM_CUDA(cudaStreamWaitEvent(p->copy_out, p->events[2 * k + 1], 0));
        CBM_CUDA(cudaMemcpy2DAsync(y + c0, pitch, p->stage_y + c0, pitch, (size_t)w * sizeof(float),
                                   (size_t)p->n_out, cudaMemcpyDeviceToHost, p->copy_out));
    }
    CBM_CUDA(cudaStreamSynchronize(p->copy_out));
    return cbm_b200_plan_status(p, s);
}

// ------------------------------------------------------------------------------------------
// Product without any allocation in the call path.
//
// The ordinary product entry points grow the plan's ready-flag and partial-sum buffers with
// cudaMalloc the first time a wider operand arrives.  Some callers must never reach an allocator
// once they are running: a serving loop that has handed all device memory to its own pool, code
// that runs while a stream is being captured, a real-time path that cannot absorb the implicit
// device synchronisation of cudaMalloc/cudaFree.  For them the same kernel is offered with its
// per-call scratch (claim counters, ready flags, partial sums of long rows) carved out of one
// fixed array that lives in the library image: every GPU that loads the library holds
// CBM_B200_STATIC_SCRATCH_BYTES of it until the process exits.
//
// The array is shared by every plan and every call on a device and keeps whatever the previous
// call left in it, so each call first clears the counters and the flags it is about to use (on
// the caller's stream).  Two such calls that overlap on one GPU — different streams, or different
// host threads — race on the array; the caller has to order them.
// ------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[CBM_B200_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
unsigned char* g_static_scratch_addr[kMaxDevices] = {nullptr};

// In host code the name g_static_scratch is only a handle for the runtime, not a device address.
// The address a kernel can use is asked for once per device, with that device current.
int static_scratch_address(int device, unsigned char** out) {
    if (device < 0 || device >= kMaxDevices)
        return cbm::fail(CBM_B200_ERR_ARG, "spmm_update_static: device ordinal out of range");
    if (!g_static_scratch_addr[device]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return cbm::fail(CBM_B200_ERR_CUDA, std::string("cudaGetSymbolAddress(g_static_scratch): ") +
                                                    cudaGetErrorString(e));
        g_static_scratch_addr[device] = static_cast<unsigned char*>(ptr);
    }
    *out = g_static_scratch_addr[device];
    return CBM_B200_OK;
}

i64 round_up_256(i64 v) { return (v + 255) / 256 * 256; }

}  // namespace

extern "C" int cbm_b200_spmm_update_static(cbm_b200_plan* p, const float* x, int64_t ldx, float* y,
                                           int64_t ldy, int32_t f, int32_t normalized,
                                           void* stream) {
    const char* who = "spmm_update_static";
    if (!p) return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": NULL plan");
    int rc = check_dense(who, x, ldx, y, ldy, f);
    if (rc) return rc;
    if (!x) return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": x is NULL");
    if (normalized && !p->normalized)
        return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": plan was created without a multiplier");
    if (p->n_rows == 0) return CBM_B200_OK;

    const bool can_v4 = (f % 4 == 0) && (ldy % 4 == 0) && aligned16(y) && (ldx % 4 == 0) && aligned16(x);
    const Shape sh = pick_shape(f, p->slab_width, can_v4);
    const i64 n_units = (i64)sh.n_slabs * p->n_items;
    if (n_units >= (i64)1 << 31)
        return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": rows x column slabs exceeds 2^31 work items");
    // layout inside the fixed array: counters | ready flags | partial sums
    const i64 off_flags = 256;
    const i64 off_slots = off_flags + round_up_256(n_units * (i64)sizeof(i32));
    const i64 need = off_slots + (i64)sh.n_slabs * p->n_slots * sh.slab_w * (i64)sizeof(float);
    if (need > (i64)CBM_B200_STATIC_SCRATCH_BYTES)
        return cbm::fail(CBM_B200_ERR_ARG,
                         std::string(who) + ": this product needs " + std::to_string(need) +
                             " bytes of scratch, the fixed array holds " +
                             std::to_string((i64)CBM_B200_STATIC_SCRATCH_BYTES) +
                             "; use cbm_b200_spmm_update / cbm_b200_fused_spmm_update");

    DeviceGuard g(p->device);
    if (!g.ok) return cbm::fail(CBM_B200_ERR_CUDA, std::string(who) + ": cudaSetDevice failed");
    unsigned char* base = nullptr;
    rc = static_scratch_address(p->device, &base);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    // counters and flags must start at zero; the partial sums are written before they are read
    CBM_CUDA(cudaMemsetAsync(base, 0, (size_t)(off_flags + n_units * (i64)sizeof(i32)), s));

    KParams kp{};
    kp.desc = p->d_desc;
    kp.col = p->d_col;
    kp.val = p->d_val;
    kp.x = x;
    kp.y = y;
    kp.ldx = ldx;
    kp.ldy = ldy;
    kp.f = f;
    kp.slab_w = sh.slab_w;
    kp.n_items = p->n_items;
    kp.n_units = n_units;
    kp.scratch = reinterpret_cast<float*>(base + off_slots);
    kp.n_slots = p->n_slots;
    kp.counter = reinterpret_cast<u64*>(base);
    kp.flags = reinterpret_cast<i32*>(base + off_flags);
    kp.epoch = 1;  // flags were just cleared, so any non-zero mark will do
    kp.status = p->d_status;
    kp.mode = MODE_FUSED;
    kp.use_scale = normalized ? 1 : 0;
    kp.wait_ns = 2000000000ULL;
    int blocks = p->n_blocks > 0 ? p->n_blocks : p->sm_count * 8;
    blocks = (int)std::max<i64>(1, std::min<i64>(blocks, (n_units + 7) / 8));
    kp.n_warps = (u64)blocks * 8;
    if (sh.v4) {
        if (sh.nv == 1) return launch_rows<1, true>(kp, blocks, s);
        if (sh.nv == 2) return launch_rows<2, true>(kp, blocks, s);
        return launch_rows<4, true>(kp, blocks, s);
    }
    if (sh.nv == 1) return launch_rows<1, false>(kp, blocks, s);
    if (sh.nv == 2) return launch_rows<2, false>(kp, blocks, s);
    return launch_rows<4, false>(kp, blocks, s);
}
