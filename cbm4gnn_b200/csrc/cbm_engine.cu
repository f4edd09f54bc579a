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
#include <utility>
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
//
// A row with many delta entries is cut into segments: all but the last become PARTIAL items that
// leave their share of the gather in a scratch slot (slot index = the item's own position); the
// last segment is the row's finishing item, which adds those slots to its own share.
//
// The schedule has two parts.  Positions [0, n_prefix) hold the items that wait for nobody — first
// every PARTIAL item, then the unsplit children of the virtual root, longest first.  Positions
// [n_prefix, n_items) hold the items that may wait: finishing items of split rows and every row
// below the first level, in breadth-first order, so that whatever an item waits for has a smaller
// position.  Delta entries are stored in item order, hence consecutive items own consecutive
// entry ranges.
struct __align__(16) RowDesc {
    i32 out_row;      // row of y this item produces (local to the shard); unused if PARTIAL
    i32 parent_row;   // row of y holding the parent's finished row, -1 under the virtual root
    i32 parent_pos;   // parent's position in processing order (index of its ready flag)
    i32 info;         // bits 0-1 ITEM_* flags, bits 8-15 number of delta entries (<= 255),
                      // bits 16-31 number of PARTIAL items of this row (finishing items only)
    i32 beg;          // first delta entry of the item in the plan's col/val arrays
    i32 first_part;   // position of the row's first PARTIAL item (when there are any)
    float scale;      // s_v  = D^-1/2 of this row (1 when the plan has no multiplier)
    float inv_parent; // 1/s_u of the parent (1 when none)
};
enum : int { ITEM_PUBLISH = 1, ITEM_PARTIAL = 2, ITEM_LEN_SHIFT = 8, ITEM_NPART_SHIFT = 16 };

enum Mode : int { MODE_FUSED = 0, MODE_DELTA_ONLY = 1, MODE_UPDATE_ONLY = 2 };

struct KParams {
    const RowDesc* desc;
    const i32* col;
    const float* val;
    const float* x;
    float* y;
    i64 ldx, ldy;
    i32 f;
    i32 slab_w;      // columns per slab
    i32 n_items;     // work items per slab
    i32 n_prefix;    // items that never wait (claimed `group` at a time)
    i32 group;       // prefix items per claim
    i32 n_pclaims;   // ceil(n_prefix / group)
    i32 claims_per_slab;  // n_pclaims + (n_items - n_prefix)
    i64 n_claims;    // claims_per_slab * n_slabs
    float* scratch;  // n_slabs * n_partial * slab_w floats: partial sums of long rows
    i32 n_partial;   // PARTIAL items (positions [0, n_partial))
    u64* counter;    // [0] next claim, [1] warps that have left; both 0 between launches
    u64 n_warps;     // warps in this launch
    i32* flags;      // n_slabs * n_items ready flags holding the epoch of the launch that set them
    i32 epoch;
    i32* status;     // 0 ok; non-zero: a wait gave up
    i32 mode;
    i32 use_scale;
    u64 wait_ns;
    // Broadcast epilogue (multi-GPU): every finished row is also written, after the optional
    // ReLU, to n_bcast further buffers with the layout of y — the slices that this shard occupies
    // in the gathered layer output of each GPU (peer memory mapped into this process, reached
    // by ordinary stores over NVLink).  y itself keeps the row as the tree needs it.
    float* bcast[CBM_B200_MAX_BCAST];
    i32 n_bcast;
    i32 bcast_relu;
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
    // The same fetch without the predicate, for slabs in which every lane has columns.
    static __device__ __forceinline__ T ld_ro(const float* p) {
        T v;
        asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                     : "l"(p));
        return v;
    }
    static __device__ __forceinline__ T ld_l2(const float* p) { return __ldcg((const float4*)p); }
    // L2-only fetch (data written earlier in the same launch), zeros when `on` is false; volatile
    // asm for the same reason as ld_ro_if.
    static __device__ __forceinline__ T ld_l2_if(const float* p, bool on) {
        T v;
        asm volatile(
            "{\n\t.reg .pred q;\n\tsetp.ne.s32 q, %5, 0;\n\t"
            "mov.f32 %0, 0f00000000;\n\tmov.f32 %1, 0f00000000;\n\t"
            "mov.f32 %2, 0f00000000;\n\tmov.f32 %3, 0f00000000;\n\t"
            "@q ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];\n\t}"
            : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
            : "l"(p), "r"((int)on)
            : "memory");
        return v;
    }
    static __device__ __forceinline__ void st(float* p, T v) { *(float4*)p = v; }
    static __device__ __forceinline__ void st_stream(float* p, T v) { __stcs((float4*)p, v); }
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
    static __device__ __forceinline__ T relu(T a) {
        a.x = fmaxf(a.x, 0.f);
        a.y = fmaxf(a.y, 0.f);
        a.z = fmaxf(a.z, 0.f);
        a.w = fmaxf(a.w, 0.f);
        return a;
    }
};
template <>
struct Vec<false> {
    using T = float;
    static constexpr int E = 1;
    static __device__ __forceinline__ T zero() { return 0.f; }
    static __device__ __forceinline__ T ld_ro_if(const float* p, bool on) {
        T v;
        asm volatile(
            "{\n\t.reg .pred q;\n\tsetp.ne.s32 q, %2, 0;\n\tmov.f32 %0, 0f00000000;\n\t"
            "@q ld.global.nc.f32 %0, [%1];\n\t}"
            : "=f"(v)
            : "l"(p), "r"((int)on));
        return v;
    }
    static __device__ __forceinline__ T ld_ro(const float* p) {
        T v;
        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
        return v;
    }
    static __device__ __forceinline__ T ld_l2(const float* p) { return __ldcg(p); }
    static __device__ __forceinline__ T ld_l2_if(const float* p, bool on) {
        T v;
        asm volatile(
            "{\n\t.reg .pred q;\n\tsetp.ne.s32 q, %2, 0;\n\tmov.f32 %0, 0f00000000;\n\t"
            "@q ld.global.cg.f32 %0, [%1];\n\t}"
            : "=f"(v)
            : "l"(p), "r"((int)on)
            : "memory");
        return v;
    }
    static __device__ __forceinline__ void st(float* p, T v) { *p = v; }
    static __device__ __forceinline__ void st_stream(float* p, T v) { __stcs(p, v); }
    static __device__ __forceinline__ T fma(float w, T a, T c) { return fmaf(w, a, c); }
    static __device__ __forceinline__ T mul(float w, T a) { return w * a; }
    static __device__ __forceinline__ T relu(T a) { return fmaxf(a, 0.f); }
};

// acc[v] += sum over entries [beg,end) of val * X[col, slab columns of this lane].
// The 32 lanes fetch 32 (col, val) pairs at once and pass them round by shuffle.  Row fetches are
// issued UNROLL at a time so that several independent loads per lane are in flight; the weights
// are picked up after the fetches have been issued.
template <int NV, bool V4, int UNROLL, bool FULL = false>
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
                for (int v = 0; v < NV; ++v) {
                    if constexpr (FULL) t[k][v] = V::ld_ro(r + v * STEP);  // every lane has columns
                    else t[k][v] = V::ld_ro_if(r + v * STEP, ok[v]);
                }
            }
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                const float w = __shfl_sync(0xffffffffu, mw, j + k);
#pragma unroll
                for (int v = 0; v < NV; ++v) acc[v] = V::fma(w, t[k][v], acc[v]);
            }
        }
        if (j < n_here) {  // the last, shorter batch: same code with the surplus fetches switched off
            T t[UNROLL][NV];
            const i32 live = n_here - j;
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                const i32 c = __shfl_sync(0xffffffffu, mc, (j + k) & 31);
                const float* r = xs + (i64)c * ldx;
#pragma unroll
                for (int v = 0; v < NV; ++v) t[k][v] = V::ld_ro_if(r + v * STEP, ok[v] && k < live);
            }
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                const float w = __shfl_sync(0xffffffffu, mw, (j + k) & 31);  // 0 past the end
#pragma unroll
                for (int v = 0; v < NV; ++v) acc[v] = V::fma(k < live ? w : 0.f, t[k][v], acc[v]);
            }
        }
    }
}

// The same sum for slabs of at most 64 columns (128-bit path): a row piece needs only 16 lanes, so
// the two half-warps fetch two different delta entries at a time and their partial sums are
// combined with one shuffle at the end.  Every lane ends up holding the total of its column group.
template <int UNROLL>
__device__ __forceinline__ void gather_row_half(const i32* __restrict__ col,
                                                const float* __restrict__ val, i32 beg, i32 end,
                                                const float* __restrict__ x_slab, i64 ldx, i32 wcols,
                                                float4& acc, int lane) {
    using V = Vec<true>;
    const int li = lane & 15, half = lane >> 4;
    const bool okh = li * 4 < wcols;
    const float* xs = x_slab + li * 4;
    for (i32 b = beg; b < end; b += 32) {
        const i32 n_here = min(32, end - b);
        i32 mc = 0;
        float mw = 0.f;
        if (lane < n_here) {
            mc = __ldg(col + b + lane);
            mw = __ldg(val + b + lane);
        }
        for (i32 j = 0; j < n_here; j += 2 * UNROLL) {
            float4 t[UNROLL];
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                const i32 idx = j + 2 * k + half;
                const i32 c = __shfl_sync(0xffffffffu, mc, idx & 31);
                t[k] = V::ld_ro_if(xs + (i64)c * ldx, okh && idx < n_here);
            }
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                const i32 idx = j + 2 * k + half;
                const float w = __shfl_sync(0xffffffffu, mw, idx & 31);
                acc = V::fma(idx < n_here ? w : 0.f, t[k], acc);
            }
        }
    }
    acc.x += __shfl_xor_sync(0xffffffffu, acc.x, 16);
    acc.y += __shfl_xor_sync(0xffffffffu, acc.y, 16);
    acc.z += __shfl_xor_sync(0xffffffffu, acc.z, 16);
    acc.w += __shfl_xor_sync(0xffffffffu, acc.w, 16);
}

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

// Maps a claim number to (slab, first item, item count): inside a slab the prefix is handed out
// `group` items at a time, the rest one item at a time.  Only items that never wait are grouped:
// a warp that sits on an item waiting for a neighbour would starve the items behind it in its
// group, which others in turn wait for (measured: 16x slower with 4 mixed items per claim).
__device__ __forceinline__ void decode_claim(const KParams& p, u64 t, i32& slab, i32& first, i32& count) {
    const unsigned u = (unsigned)t;  // the host refuses launches of 2^31 claims or more
    slab = (i32)(u / (unsigned)p.claims_per_slab);
    const i32 r = (i32)(u - (unsigned)slab * (unsigned)p.claims_per_slab);
    if (r < p.n_pclaims) {
        first = r * p.group;
        count = min(p.group, p.n_prefix - first);
    } else {
        first = p.n_prefix + (r - p.n_pclaims);
        count = 1;
    }
}

// Everything that happens to an item once its own gather is in `acc`: park a PARTIAL share, or
// collect the row's parked shares, add the parent's finished row, scale, store and publish.
// Returns false when a bounded wait ran out.
template <int NV, bool V4>
__device__ __forceinline__ bool finish_item(const KParams& p, i32 slab, i32 pos, i32 out_row,
                                            i32 parent_row, i32 parent_pos, i32 info,
                                            i32 first_part, float scale, float inv_parent,
                                            typename Vec<V4>::T (&acc)[NV], const bool (&ok)[NV],
                                            i32 c0, int lane) {
    using V = Vec<V4>;
    constexpr int STEP = 32 * V::E;
    i32* slab_flags = p.flags + (i64)slab * p.n_items;
    if (info & ITEM_PARTIAL) {
        float* slot = p.scratch + ((i64)slab * p.n_partial + pos) * p.slab_w + lane * V::E;
#pragma unroll
        for (int v = 0; v < NV; ++v)
            if (ok[v]) V::st(slot + v * STEP, acc[v]);
        // the warp barrier orders every lane's stores before lane 0's release store, whose
        // gpu-scope release then covers them all: no per-lane fence is needed
        __syncwarp();
        if (lane == 0) st_release(slab_flags + pos, p.epoch);
        return true;
    }
    const i32 n_part = (i32)((unsigned)info >> ITEM_NPART_SHIFT);
    if (n_part > 0 && p.mode != MODE_UPDATE_ONLY) {
        // A row can have hundreds of parked shares; taking them one memory round trip at a time
        // would serialise the whole product behind the longest row.  The 32 lanes wait for 32
        // flags at once, then the shares are fetched PART_BATCH at a time and added in slot order
        // (a fixed order, so results do not depend on timing).
        bool mine = true;
        for (i32 k = lane; k < n_part; k += 32)
            mine = mine && wait_ready(slab_flags + first_part + k, p.epoch, p.status, p.wait_ns);
        if (!__all_sync(0xffffffffu, mine)) return false;
        // lane k acquired flag k; the warp barrier extends that ordering to the lanes that did not
        __syncwarp();
        constexpr int PART_BATCH = NV == 1 ? 8 : 4;
        const float* slot0 = p.scratch + ((i64)slab * p.n_partial + first_part) * p.slab_w + lane * V::E;
        for (i32 k = 0; k < n_part; k += PART_BATCH) {
            typename V::T t[PART_BATCH][NV];
#pragma unroll
            for (int j = 0; j < PART_BATCH; ++j)
#pragma unroll
                for (int v = 0; v < NV; ++v)
                    t[j][v] = V::ld_l2_if(slot0 + (i64)(k + j) * p.slab_w + v * STEP, ok[v] && (k + j) < n_part);
#pragma unroll
            for (int j = 0; j < PART_BATCH; ++j)
#pragma unroll
                for (int v = 0; v < NV; ++v) acc[v] = V::fma(1.0f, t[j][v], acc[v]);
        }
    }
    const i32 lane_col = c0 + lane * V::E;
    if (p.mode != MODE_DELTA_ONLY) {
        if (parent_row >= 0) {
            if (!wait_ready(slab_flags + parent_pos, p.epoch, p.status, p.wait_ns)) return false;
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
    float* yrow = p.y + (i64)out_row * p.ldy + lane_col;
    if (info & ITEM_PUBLISH) {
#pragma unroll
        for (int v = 0; v < NV; ++v)
            if (ok[v]) V::st(yrow + v * STEP, acc[v]);
    } else {
        // nobody reads this row again during the product: a streaming store keeps it from
        // pushing slabs of X out of L2
#pragma unroll
        for (int v = 0; v < NV; ++v)
            if (ok[v]) V::st_stream(yrow + v * STEP, acc[v]);
    }
    if ((info & ITEM_PUBLISH) && p.mode != MODE_DELTA_ONLY) {
        __syncwarp();
        if (lane == 0) st_release(slab_flags + pos, p.epoch);
    }
    if (p.n_bcast > 0) {
        if (p.bcast_relu) {
#pragma unroll
            for (int v = 0; v < NV; ++v) acc[v] = V::relu(acc[v]);
        }
        const i64 off = (i64)out_row * p.ldy + lane_col;
        for (int k = 0; k < p.n_bcast; ++k) {
            float* dst = p.bcast[k] + off;
#pragma unroll
            for (int v = 0; v < NV; ++v)
                if (ok[v]) V::st(dst + v * STEP, acc[v]);
        }
    }
    return true;
}

// Product kernel, register form: one warp per (item, column slab), the gather held in registers.
// Serves operands the bulk-copy form cannot take (width not a multiple of 4 floats, unaligned
// pointers) and the update-only mode, which gathers nothing; it is also the default form.
// UNROLL = row fetches in flight per lane, MINB = thread blocks the register budget must allow
// per SM.
template <int NV, bool V4, int UNROLL, int MINB>
__global__ void __launch_bounds__(256, MINB) cbm_items_kernel(const KParams p) {
    using V = Vec<V4>;
    using T = typename V::T;
    constexpr int STEP = 32 * V::E;
    const int lane = threadIdx.x & 31;
    for (;;) {
        u64 t = 0;
        if (lane == 0) t = atomicAdd(p.counter, 1ULL);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (t >= (u64)p.n_claims) {
            leave(p, lane);
            return;
        }
        i32 slab, first, count;
        decode_claim(p, t, slab, first, count);
        const i32 c0 = slab * p.slab_w;
        const i32 wcols = min(p.slab_w, p.f - c0);
        bool ok[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) ok[v] = (lane * V::E + v * STEP) < wcols;
        for (i32 pos = first; pos < first + count; ++pos) {
            const int4 da = __ldg((const int4*)(p.desc + pos));
            const int4 db = __ldg((const int4*)(p.desc + pos) + 1);
            const i32 info = da.w;
            if ((info & ITEM_PARTIAL) && p.mode == MODE_UPDATE_ONLY) continue;  // nothing to gather
            T acc[NV];
            if (p.mode == MODE_UPDATE_ONLY) {
                const float* yrow = p.y + (i64)da.x * p.ldy + c0 + lane * V::E;
#pragma unroll
                for (int v = 0; v < NV; ++v) acc[v] = ok[v] ? V::ld_l2(yrow + v * STEP) : V::zero();
            } else {
#pragma unroll
                for (int v = 0; v < NV; ++v) acc[v] = V::zero();
                const i32 len = (info >> ITEM_LEN_SHIFT) & 0xff;
                if constexpr (V4 && NV == 1) {
                    if (wcols <= 64)
                        gather_row_half<UNROLL>(p.col, p.val, db.x, db.x + len, p.x + c0, p.ldx, wcols, acc[0], lane);
                    else if (wcols == 128)  // a complete slab: no per-lane predicate on the fetches
                        gather_row<NV, V4, UNROLL, true>(p.col, p.val, db.x, db.x + len, p.x + c0 + lane * V::E,
                                                         p.ldx, ok, acc, lane);
                    else
                        gather_row<NV, V4, UNROLL>(p.col, p.val, db.x, db.x + len, p.x + c0 + lane * V::E,
                                                   p.ldx, ok, acc, lane);
                } else {
                    gather_row<NV, V4, UNROLL>(p.col, p.val, db.x, db.x + len, p.x + c0 + lane * V::E, p.ldx,
                                               ok, acc, lane);
                }
            }
            if (!finish_item<NV, V4>(p, slab, pos, da.x, da.y, da.z, info, db.y, __int_as_float(db.z),
                                     __int_as_float(db.w), acc, ok, c0, lane)) {
                leave(p, lane);
                return;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Bulk-copy form of the product kernel.
//
// The register form keeps at most UNROLL row fetches per lane in flight, so a typical row of 20-30
// delta entries costs several memory round trips in a row, on top of the round trips for the
// claim, the descriptor and the indices.  Here each lane issues ONE bulk asynchronous copy
// (cp.async.bulk, the untiled TMA path) that brings a whole slab-wide piece of one operand row
// into shared memory, so up to NB rows per stage are in flight per warp and complete on an
// mbarrier; stages alternate so the next batch is on its way while the current one is summed out
// of shared memory.  Items of the never-waiting prefix are claimed `group` at a time and their
// consecutive entry ranges are streamed as one sequence of batches, which amortises the claim and
// keeps short rows from leaving the pipeline empty.
//
// Measured on B200 (100 000-row product, F = 500): the copy engine retires about 7 G bulk copies
// per second whatever their size between 512 B and 1 KB, so 512-byte pieces reach 3.5 TB/s and
// 1 KB pieces 7 TB/s, against 12.8 TB/s for the register form.  Row pieces of a few hundred bytes
// are too small for this path; it is kept as an opt-in form (cbm_b200_plan_tune, form = 1) and the
// register form is the default.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_addr(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded: gives up after two seconds (each poll itself blocks for a hardware-defined slice).
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, i32* status) {
    if (mbar_try_wait(bar, parity)) return true;
    const u64 t0 = global_ns();
    for (unsigned spins = 0; spins < (1u << 24); ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 63u) == 63u && global_ns() - t0 > 2000000000ULL) break;
    }
    atomicExch(status, CBM_B200_ERR_TIMEOUT);
    return false;
}
// One row piece global -> shared; src, dst and bytes are multiples of 16 (the host checks).
__device__ __forceinline__ void bulk_copy_g2s(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void fence_async_proxy() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

template <int SLABW, int NB, int STAGES>
struct TmaLayout {
    static constexpr int SLABB = SLABW * 4;                   // bytes of one row piece
    static constexpr int STAGE_BYTES = NB * SLABB;            // NB row pieces
    // rounded up so that every warp's area starts 128-byte aligned (bulk copies need 16)
    static constexpr int WARP_BYTES = (STAGES * STAGE_BYTES + STAGES * NB * 4 + STAGES * 8 + 127) / 128 * 128;
    static __host__ __device__ constexpr int smem_bytes(int warps) { return warps * WARP_BYTES; }
};

template <int SLABW, int NB, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1) cbm_items_tma_kernel(const KParams p) {
    using V = Vec<true>;
    using T = float4;
    using L = TmaLayout<SLABW, NB, STAGES>;
    constexpr int NV = SLABW / 128;
    constexpr int STEP = 128;
    static_assert(NB <= 32 && SLABW % 128 == 0, "one lane per staged row; slabs of 128 floats");
    extern __shared__ __align__(128) unsigned char smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    unsigned char* my = smem + (size_t)warp * L::WARP_BYTES;
    unsigned char* rows = my;                                               // [STAGES][NB][SLABB]
    float* wts = reinterpret_cast<float*>(my + STAGES * L::STAGE_BYTES);    // [STAGES][NB]
    const unsigned bar0 = smem_addr(my + STAGES * L::STAGE_BYTES + STAGES * NB * 4);
    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_async_proxy();
    __syncwarp();
    unsigned parity = 0;  // bit s = phase the next wait on stage s looks for

    for (;;) {
        u64 t = 0;
        if (lane == 0) t = atomicAdd(p.counter, 1ULL);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (t >= (u64)p.n_claims) {
            leave(p, lane);
            return;
        }
        i32 slab, first, count;
        decode_claim(p, t, slab, first, count);
        const i32 c0 = slab * SLABW;
        const i32 wcols = min(SLABW, p.f - c0);
        const unsigned piece = (unsigned)wcols * 4u;
        bool ok[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) ok[v] = (lane * 4 + v * STEP) < wcols;

        // lane i keeps the descriptor of item first + i
        int4 da = make_int4(0, -1, -1, 0), db = make_int4(0, 0, 0, 0);
        if (lane < count) {
            da = __ldg((const int4*)(p.desc + first + lane));
            db = __ldg((const int4*)(p.desc + first + lane) + 1);
        }
        const i32 my_end = db.x + ((da.w >> ITEM_LEN_SHIFT) & 0xff);
        const i32 e_begin = __shfl_sync(0xffffffffu, db.x, 0);
        const i32 e_end = __shfl_sync(0xffffffffu, my_end, count - 1);
        const i32 n_batches = (e_end - e_begin + NB - 1) / NB;
        const float* xs = p.x + c0;

        // indices of batch q, one entry per lane
        auto load_idx = [&](i32 q, i32& c, float& w) {
            const i32 e = e_begin + q * NB + lane;
            c = -1;
            w = 0.f;
            if (lane < NB && e < e_end) {
                c = __ldg(p.col + e);
                w = __ldg(p.val + e);
            }
        };
        // start the copies of batch q into its stage
        auto issue = [&](i32 q, i32 c, float w) {
            const int s = q % STAGES;
            const i32 cnt = min(NB, e_end - (e_begin + q * NB));
            const unsigned bar = bar0 + 8 * s;
            __syncwarp();         // every lane has finished reading this stage
            fence_async_proxy();  // ... before the copies of the async proxy may land in it
            if (lane == 0) mbar_expect_tx(bar, (unsigned)cnt * piece);
            if (lane < NB) wts[s * NB + lane] = w;
            __syncwarp();
            if (lane < cnt)
                bulk_copy_g2s(smem_addr(rows + (size_t)s * L::STAGE_BYTES + (size_t)lane * L::SLABB),
                              xs + (i64)c * p.ldx, piece, bar);
        };

        T acc[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[v] = V::zero();
        i32 cur = 0;  // item being accumulated
        i32 cur_end = __shfl_sync(0xffffffffu, my_end, 0);
        bool alive = true;
        auto flush = [&](i32 i) {  // finish item first + i with what is in acc, then clear acc
            const i32 o = __shfl_sync(0xffffffffu, da.x, i), pr = __shfl_sync(0xffffffffu, da.y, i);
            const i32 pp = __shfl_sync(0xffffffffu, da.z, i), inf = __shfl_sync(0xffffffffu, da.w, i);
            const i32 fp = __shfl_sync(0xffffffffu, db.y, i);
            const float sc = __int_as_float(__shfl_sync(0xffffffffu, db.z, i));
            const float ip = __int_as_float(__shfl_sync(0xffffffffu, db.w, i));
            alive = finish_item<NV, true>(p, slab, first + i, o, pr, pp, inf, fp, sc, ip, acc, ok, c0, lane);
#pragma unroll
            for (int v = 0; v < NV; ++v) acc[v] = V::zero();
        };

        i32 c_nx = -1;
        float w_nx = 0.f;
        i32 issued = 0;
        if (n_batches > 0) {
            load_idx(0, c_nx, w_nx);
            issue(0, c_nx, w_nx);
            issued = 1;
            if (n_batches > 1) load_idx(1, c_nx, w_nx);
        }
        i32 waited = 0;  // batches whose arrival has been consumed
        for (i32 q = 0; q < n_batches && alive; ++q) {
            while (issued < n_batches && issued - q < STAGES) {  // keep the other stages busy
                issue(issued, c_nx, w_nx);
                ++issued;
                if (issued < n_batches) load_idx(issued, c_nx, w_nx);
            }
            const int s = q % STAGES;
            if (!mbar_wait(bar0 + 8 * s, (parity >> s) & 1u, p.status)) {
                alive = false;
                break;
            }
            parity ^= 1u << s;
            waited = q + 1;
            const i32 e0 = e_begin + q * NB;
            const i32 cnt = min(NB, e_end - e0);
            const unsigned char* st = rows + (size_t)s * L::STAGE_BYTES + lane * 16;
            const float* wq = wts + s * NB;
            for (i32 l = 0; l < cnt && alive; ++l) {
                while (e0 + l == cur_end && cur < count - 1 && alive) {  // entry belongs to a later item
                    flush(cur);
                    ++cur;
                    cur_end = __shfl_sync(0xffffffffu, my_end, cur);
                }
                const float w = wq[l];
#pragma unroll
                for (int v = 0; v < NV; ++v)
                    if (ok[v])
                        acc[v] = V::fma(w, *reinterpret_cast<const float4*>(st + (size_t)l * L::SLABB + v * 512),
                                        acc[v]);
            }
        }
        if (!alive) {
            // A wait ran out: the status word is set.  Copies already issued into this warp's
            // shared-memory stages must land before the block may retire and its shared memory
            // be handed on, so every outstanding stage is waited for (bounded) and discarded.
            for (i32 qq = waited; qq < issued; ++qq) {
                const int s2 = qq % STAGES;
                mbar_wait(bar0 + 8 * s2, (parity >> s2) & 1u, p.status);
                parity ^= 1u << s2;
            }
            leave(p, lane);
            return;
        }
        while (cur < count && alive) {  // the last item, and any empty items behind it
            flush(cur);
            ++cur;
        }
        if (!alive) {
            leave(p, lane);
            return;
        }
    }
}

// Plain CSR product (no tree): rows in natural order, one warp per (row, slab), grid-stride.
template <int NV, bool V4>
__global__ void __launch_bounds__(256, (NV >= 4 ? 2 : 3))
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
        gather_row<NV, V4, (NV == 1 ? 8 : 4)>(col, val, __ldg(row_b + row), __ldg(row_e + row), x + lane_col, ldx, ok,
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
// Default slab width of the 128-bit path: 128 columns, one 16-byte vector per lane.  One slab of the
// operand (n_labels rows of slab_w floats) is what every row gathers from while that slab is
// processed, and it should stay in L2.  B200's 126 MB L2 is two partitions that each keep their own
// copy of lines read from both dies, so about half of it holds such an operand: at 100 000 rows a
// 256-column slab (102 MB) does not stay, a 128-column slab (51 MB) does, and DRAM traffic halves.
// Measured on B200, 128 columns also win where no slab can stay resident (200 000 - 400 000 rows:
// 0.55 / 0.71 ms against 0.63 / 0.77 ms for 256 columns; 236 000 rows, width 256: 0.307 against
// 0.324 ms): the one-vector form holds eight row fetches per lane in 56 registers and keeps 32 warps
// per SM, the two-vector form four fetches in 72 registers and 24 warps.
i32 default_slab_v4(i64 /*n_labels*/) { return 128; }

Shape pick_shape(i32 f, i32 want_slab, bool can_v4, i64 n_labels) {
    Shape s{};
    s.v4 = can_v4;
    const i32 lane_w = s.v4 ? 128 : 32;  // columns covered by one vector per lane
    i32 slab = want_slab > 0 ? want_slab : (s.v4 ? default_slab_v4(n_labels) : 64);
    if (s.v4 && (want_slab == 64 || want_slab == 32)) {  // narrow slabs on request: half-warp gather
        s.nv = 1;
        s.slab_w = want_slab;
        s.n_slabs = (f + want_slab - 1) / want_slab;
        return s;
    }
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
    i32 n_prefix = 0;  // items that never wait
    i32 n_partial = 0; // PARTIAL items = scratch slots per slab
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
    i32 form = 0;      // 0 register form, 1 bulk-copy form
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

namespace {

// The host-side schedule of one plan, before anything touches the device.
struct Schedule {
    std::vector<RowDesc> desc;
    std::vector<i32> pcol;
    std::vector<float> pval;
    i32 n_prefix = 0, n_partial = 0, n_rows_owned = 0, depth = 0, n_root_children = 0, n_labels = 0;
};

// Checks, before any launch, the properties the kernels rely on: items wait only for smaller
// positions (so the in-order claiming cannot deadlock), whoever is waited for publishes, entry
// ranges are consecutive, every output row is produced exactly once and every parked share is
// collected exactly once.
int validate_schedule(const Schedule& sch, i32 n_out) {
    const i32 n_items = (i32)sch.desc.size();
    auto bad = [](const char* what) { return cbm::fail(CBM_B200_ERR_FORMAT, std::string("schedule check: ") + what); };
    if (sch.n_partial > sch.n_prefix || sch.n_prefix > n_items) return bad("prefix bounds");
    std::vector<char> produced((size_t)std::max(n_out, 0), 0), collected((size_t)sch.n_partial, 0);
    i64 cursor = 0;
    for (i32 pos = 0; pos < n_items; ++pos) {
        const RowDesc& d = sch.desc[pos];
        const i32 len = (d.info >> ITEM_LEN_SHIFT) & 0xff;
        const i32 n_part = (i32)((unsigned)d.info >> ITEM_NPART_SHIFT);
        const bool partial = (d.info & ITEM_PARTIAL) != 0;
        if (d.beg != cursor) return bad("entry ranges are not consecutive");
        cursor += len;
        if (partial != (pos < sch.n_partial)) return bad("PARTIAL items must fill positions [0, n_partial)");
        if (partial) {
            if (!(d.info & ITEM_PUBLISH) || d.parent_row >= 0 || n_part != 0) return bad("malformed PARTIAL item");
            continue;
        }
        if (d.out_row < 0 || d.out_row >= n_out || produced[d.out_row]) return bad("output row missing or produced twice");
        produced[d.out_row] = 1;
        if (pos < sch.n_prefix && (d.parent_row >= 0 || n_part != 0)) return bad("a prefix item would have to wait");
        if (d.parent_row >= 0) {
            if (d.parent_pos < 0 || d.parent_pos >= pos) return bad("an item waits for a later position");
            const RowDesc& q = sch.desc[d.parent_pos];
            if ((q.info & ITEM_PARTIAL) || !(q.info & ITEM_PUBLISH) || q.out_row != d.parent_row)
                return bad("parent item does not publish the row its child reads");
        }
        if (n_part > 0) {
            if (pos < sch.n_prefix || d.first_part < 0 || d.first_part + n_part > sch.n_partial)
                return bad("parked shares out of range");
            for (i32 k = 0; k < n_part; ++k) {
                if (collected[d.first_part + k]) return bad("a parked share is collected twice");
                collected[d.first_part + k] = 1;
            }
        }
    }
    if (cursor != (i64)sch.pcol.size() || sch.pcol.size() != sch.pval.size()) return bad("entries not covered exactly once");
    for (char c : collected)
        if (!c) return bad("a parked share is never collected");
    i32 rows = 0;
    for (char c : produced) rows += c;
    if (rows != sch.n_rows_owned) return bad("owned rows and produced rows differ");
    return CBM_B200_OK;
}

// csr_cols > 0 schedules a plain CSR matrix with that many columns (no tree: every row hangs off
// the virtual root, mst_row / mst_col / perm are not read); csr_cols == 0 schedules a CBM structure.
int build_schedule(int32_t n, const int32_t* mst_row, const int32_t* mst_col, const int32_t* delta_crow,
                   const int32_t* delta_col, const float* delta_val, const float* multiplier,
                   const int32_t* perm, int32_t n_labels, int32_t own_begin, int32_t own_end, Schedule& sch,
                   int32_t csr_cols = 0) {
    std::vector<i32> flat_row, flat_col;
    if (csr_cols > 0) {
        if (n < 0 || !delta_crow) return cbm::fail(CBM_B200_ERR_ARG, "csr_plan_create: NULL row pointers");
        flat_row.assign((size_t)n + 2, 0);
        flat_row[(size_t)n + 1] = n;
        flat_col.resize((size_t)n);
        for (i32 v = 0; v < n; ++v) flat_col[v] = v;
        mst_row = flat_row.data();
        mst_col = flat_col.data();
        perm = nullptr;
        n_labels = n;  // labels of the rows; the column bound is csr_cols
        own_begin = 0;
        own_end = n;
    }
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
    const i32 col_bound = csr_cols > 0 ? csr_cols : n;

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
        if (delta_col[k] < 0 || delta_col[k] >= col_bound)
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

    // ---- schedule (layout described at RowDesc) ----
    const i32 SEG = 128;         // delta entries per item of a split row
    const i32 SPLIT_OVER = 192;  // rows longer than this are split
    auto row_len = [&](i32 v) { return delta_crow[v + 1] - delta_crow[v]; };
    auto is_split = [&](i32 v) { return row_len(v) > SPLIT_OVER; };
    std::vector<i32> owned_rows;  // breadth-first
    owned_rows.reserve((size_t)(own_end - own_begin));
    for (i32 v : order)
        if (owned(v)) {
            const i32 u = parent[v];
            if (u != n && !owned(u))
                return cbm::fail(CBM_B200_ERR_ARG,
                                 "plan_create: owned range cuts a subtree (parent of an owned row "
                                 "is not owned)");
            owned_rows.push_back(v);
        }
    std::vector<RowDesc>& desc = sch.desc;
    std::vector<i32>& pcol = sch.pcol;
    std::vector<float>& pval = sch.pval;
    pcol.reserve((size_t)nd_all);
    pval.reserve((size_t)nd_all);
    auto append_entries = [&](i32 v, i32 from, i32 to) {  // entries [from, to) of row v
        const i32 beg = (i32)pcol.size();
        for (i32 k = delta_crow[v] + from; k < delta_crow[v] + to; ++k) {
            pcol.push_back(label(delta_col[k]));
            pval.push_back(delta_val[k]);
        }
        return beg;
    };
    // 1. PARTIAL items of every split row
    std::vector<i32> first_part((size_t)n, -1);
    for (i32 v : owned_rows) {
        if (!is_split(v)) continue;
        const i32 n_part = (row_len(v) + SEG - 1) / SEG - 1;
        if (n_part > 0xffff)
            return cbm::fail(CBM_B200_ERR_ARG, "plan_create: a row has more than 8388480 delta entries");
        first_part[v] = (i32)desc.size();
        for (i32 k = 0; k < n_part; ++k) {
            RowDesc q{};
            q.out_row = 0;
            q.parent_row = -1;
            q.parent_pos = -1;
            q.info = ITEM_PARTIAL | ITEM_PUBLISH | (SEG << ITEM_LEN_SHIFT);
            q.beg = append_entries(v, k * SEG, (k + 1) * SEG);
            q.first_part = -1;
            q.scale = 1.0f;
            q.inv_parent = 1.0f;
            desc.push_back(q);
        }
    }
    const i32 n_partial = (i32)desc.size();
    // 2. unsplit children of the virtual root, longest first
    std::vector<i32> pos_of((size_t)n, -1);
    i32 depth = 0, n_root_children = 0;
    auto add_row_item = [&](i32 v) {
        const i32 u = parent[v];
        const i32 len = row_len(v);
        const i32 n_part = is_split(v) ? (len + SEG - 1) / SEG - 1 : 0;
        RowDesc d{};
        d.out_row = label(v) - own_begin;
        d.parent_row = (u == n) ? -1 : label(u) - own_begin;
        d.parent_pos = (u == n) ? -1 : pos_of[u];
        d.beg = append_entries(v, n_part * SEG, len);
        d.info = ((len - n_part * SEG) << ITEM_LEN_SHIFT) | (n_part << ITEM_NPART_SHIFT);
        d.first_part = first_part[v];
        d.scale = multiplier ? multiplier[v] : 1.0f;
        d.inv_parent = (multiplier && u != n) ? 1.0f / multiplier[u] : 1.0f;
        pos_of[v] = (i32)desc.size();
        if (u != n) desc[pos_of[u]].info |= ITEM_PUBLISH;
        else ++n_root_children;
        depth = std::max(depth, level[v]);
        desc.push_back(d);
    };
    {
        std::vector<i32> easy;
        for (i32 v : owned_rows)
            if (parent[v] == n && !is_split(v)) easy.push_back(v);
        std::stable_sort(easy.begin(), easy.end(), [&](i32 a, i32 b) { return row_len(a) > row_len(b); });
        for (i32 v : easy) add_row_item(v);
    }
    const i32 n_prefix = (i32)desc.size();
    // 3. everything that may wait, breadth-first: finishing items of split rows, rows with a parent
    for (i32 v : owned_rows)
        if (parent[v] != n || is_split(v)) add_row_item(v);
    sch.n_rows_owned = (i32)owned_rows.size();
    sch.n_prefix = n_prefix;
    sch.n_partial = n_partial;
    sch.depth = depth;
    sch.n_root_children = n_root_children;
    sch.n_labels = csr_cols > 0 ? csr_cols : n_labels;
    return validate_schedule(sch, own_end - own_begin);
}


}  // namespace

extern "C" int cbm_b200_schedule_info(int32_t n, const int32_t* mst_row, const int32_t* mst_col,
                                      const int32_t* delta_crow, const int32_t* delta_col,
                                      const float* delta_val, const float* multiplier,
                                      const int32_t* perm, int32_t n_labels, int32_t own_begin,
                                      int32_t own_end, int32_t* n_items, int32_t* n_prefix,
                                      int32_t* n_partial, int32_t* n_rows) {
    Schedule sch;
    const int rc = build_schedule(n, mst_row, mst_col, delta_crow, delta_col, delta_val, multiplier, perm,
                                  n_labels, own_begin, own_end, sch);
    if (rc) return rc;
    if (n_items) *n_items = (i32)sch.desc.size();
    if (n_prefix) *n_prefix = sch.n_prefix;
    if (n_partial) *n_partial = sch.n_partial;
    if (n_rows) *n_rows = sch.n_rows_owned;
    return CBM_B200_OK;
}

namespace {
int plan_from_schedule(Schedule& sch, int32_t n, int32_t n_out, bool normalized, int32_t device,
                       cbm_b200_plan** out);
}

extern "C" int cbm_b200_plan_create(int32_t n, const int32_t* mst_row, const int32_t* mst_col,
                                    const int32_t* delta_crow, const int32_t* delta_col,
                                    const float* delta_val, const float* multiplier,
                                    const int32_t* perm, int32_t n_labels, int32_t own_begin,
                                    int32_t own_end, int32_t device, cbm_b200_plan** out) {
    if (!out) return cbm::fail(CBM_B200_ERR_ARG, "plan_create: out is NULL");
    *out = nullptr;
    Schedule sch;
    const int rc0 = build_schedule(n, mst_row, mst_col, delta_crow, delta_col, delta_val, multiplier, perm,
                                   n_labels, own_begin, own_end, sch);
    if (rc0) return rc0;
    return plan_from_schedule(sch, n, own_end - own_begin, multiplier != nullptr, device, out);
}

extern "C" int cbm_b200_csr_plan_create(int32_t n_rows, int32_t n_cols, const int32_t* crow,
                                        const int32_t* col, const float* val, int32_t device,
                                        cbm_b200_plan** out) {
    if (!out) return cbm::fail(CBM_B200_ERR_ARG, "csr_plan_create: out is NULL");
    *out = nullptr;
    if (n_cols <= 0) return cbm::fail(CBM_B200_ERR_ARG, "csr_plan_create: n_cols must be positive");
    Schedule sch;
    const int rc0 = build_schedule(n_rows, nullptr, nullptr, crow, col, val, nullptr, nullptr, 0, 0, 0, sch, n_cols);
    if (rc0) return rc0;
    return plan_from_schedule(sch, n_rows, n_rows, false, device, out);
}

namespace {
int plan_from_schedule(Schedule& sch, int32_t n, int32_t n_out, bool normalized, int32_t device,
                       cbm_b200_plan** out) {
    const int32_t n_labels = sch.n_labels;
    std::vector<RowDesc>& desc = sch.desc;
    std::vector<i32>& pcol = sch.pcol;
    std::vector<float>& pval = sch.pval;
    const i32 n_rows_owned = sch.n_rows_owned, n_prefix = sch.n_prefix, n_partial = sch.n_partial;
    const i32 depth = sch.depth, n_root_children = sch.n_root_children;

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
    p->n_out = n_out;
    p->n_rows = n_rows_owned;
    p->n_items = (i32)desc.size();
    p->n_prefix = n_prefix;
    p->n_partial = n_partial;
    p->n_delta = (i64)pcol.size();
    p->n_root_children = n_root_children;
    p->depth = depth;
    p->normalized = normalized;
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
}  // namespace

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
                                  int32_t host_chunk, int32_t form) {
    if (!p) return cbm::fail(CBM_B200_ERR_ARG, "plan_tune: NULL plan");
    if (slab_width < 0 || n_blocks < 0 || host_chunk < 0 || form < 0 || form > 1)
        return cbm::fail(CBM_B200_ERR_ARG, "plan_tune: knob out of range");
    if (host_chunk % 4 != 0) return cbm::fail(CBM_B200_ERR_ARG, "plan_tune: host_chunk must be a multiple of 4");
    p->form = form;
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

int check_dense(const char* who, const void* x, i64 ldx, const void* y, i64 ldy, i32 f) {
    if (f <= 0) return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": f must be positive");
    if (!y || ldy < f) return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": bad y / ldy");
    if (x && ldx < f) return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": ldx < f");
    if (ldx > INT32_MAX || ldy > INT32_MAX)
        return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": leading dimension exceeds 2^31-1");
    if (x && x == y) return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": x and y alias");
    return CBM_B200_OK;
}

// How one product is cut into claims and which kernel form runs it.
struct LaunchCfg {
    Shape sh{};
    int tma = 0;       // 0: register form; otherwise the bulk-copy form (variant number)
    i32 group = 1;     // prefix items per claim
    i32 n_pclaims = 0, claims_per_slab = 0;
    i64 n_claims = 0;
    i64 need_flags = 0;        // int32 words
    i64 need_scratch = 0;      // floats
};

int plan_cfg(const cbm_b200_plan* p, const char* who, const float* x, i64 ldx, const float* y, i64 ldy,
             i32 f, int mode, LaunchCfg& c) {
    const bool can_v4 = (f % 4 == 0) && (ldy % 4 == 0) && aligned16(y) &&
                        (mode == MODE_UPDATE_ONLY || ((ldx % 4 == 0) && aligned16(x)));
    int tma = p->form;
    if (!can_v4 || mode == MODE_UPDATE_ONLY) tma = 0;
    c.tma = tma;
    if (tma) {
        const i32 slab = 256;  // 1 KB row pieces: the copy engine is bound by copies, not bytes
        c.sh.v4 = true;
        c.sh.nv = slab / 128;
        c.sh.slab_w = slab;
        c.sh.n_slabs = (f + slab - 1) / slab;
        c.group = 16;
    } else {
        c.sh = pick_shape(f, p->slab_width, can_v4, p->n_labels);
        // never-waiting items are claimed 4 at a time: measured best on B200 (fewer trips to the
        // claim counter, which bounds short-row workloads; larger groups unbalance the long rows).
        // A small product keeps single claims: with fewer claims than resident warps, grouping
        // only idles warps.
        c.group = ((i64)p->n_prefix * c.sh.n_slabs >= (i64)p->sm_count * 256) ? 4 : 1;
    }
    c.n_pclaims = (p->n_prefix + c.group - 1) / c.group;
    c.claims_per_slab = c.n_pclaims + (p->n_items - p->n_prefix);
    c.n_claims = (i64)c.claims_per_slab * c.sh.n_slabs;
    c.need_flags = (i64)c.sh.n_slabs * p->n_items;
    c.need_scratch = (i64)c.sh.n_slabs * p->n_partial * c.sh.slab_w;
    if (c.need_flags >= (i64)1 << 31)
        return cbm::fail(CBM_B200_ERR_ARG, std::string(who) + ": rows x column slabs exceeds 2^31 work items");
    return CBM_B200_OK;
}

template <int SLABW, int NB, int STAGES, int WARPS>
int launch_tma(KParams& kp, int sm_count, cudaStream_t s) {
    using L = TmaLayout<SLABW, NB, STAGES>;
    static bool configured[64] = {false};
    int dev = 0;
    CBM_CUDA(cudaGetDevice(&dev));
    auto kern = cbm_items_tma_kernel<SLABW, NB, STAGES, WARPS>;
    const int smem = L::smem_bytes(WARPS);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        CBM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[dev] = true;
    }
    const int blocks = (int)std::max<i64>(1, std::min<i64>(sm_count, (kp.n_claims + WARPS - 1) / WARPS));
    kp.n_warps = (u64)blocks * WARPS;
    kern<<<blocks, WARPS * 32, smem, s>>>(kp);
    CBM_CUDA(cudaGetLastError());
    return CBM_B200_OK;
}

template <int NV, bool V4>
int launch_regs(KParams& kp, int want_blocks, int sm_count, cudaStream_t s) {
    // Unroll depth and resident blocks per SM were chosen by measurement on B200.  For the default
    // form (one float4 per lane, 128-column slabs) 4 gathers in flight per warp at 48 resident
    // warps per SM (40 registers) beat 8 in flight at 32 warps (64 registers) by 3 % on wide
    // operands and tie on narrow ones; forms that spill registers lose more than extra resident
    // warps gain.
    constexpr int kUnroll = NV == 1 ? (V4 ? 4 : 8) : 4;
    constexpr int kResident = NV == 1 ? (V4 ? 6 : 4) : (NV == 2 ? 3 : 2);
    int blocks = want_blocks > 0 ? want_blocks : sm_count * (NV == 1 && V4 ? kResident : 8);
    blocks = (int)std::max<i64>(1, std::min<i64>(blocks, (kp.n_claims + 7) / 8));
    kp.n_warps = (u64)blocks * 8;
    cbm_items_kernel<NV, V4, kUnroll, kResident><<<blocks, 256, 0, s>>>(kp);
    CBM_CUDA(cudaGetLastError());
    return CBM_B200_OK;
}

// Fills the launch parameters that do not depend on where the scratch lives, and launches.
struct Bcast {
    int n = 0;
    int relu = 0;
    float* dst[CBM_B200_MAX_BCAST] = {nullptr};
};

int launch_plan(cbm_b200_plan* p, const LaunchCfg& c, const float* x, i64 ldx, float* y, i64 ldy, i32 f,
                int mode, bool use_scale, u64* counter, i32* flags, float* scratch, i32 epoch,
                cudaStream_t s, const Bcast* bc = nullptr) {
    KParams kp{};
    if (bc) {
        kp.n_bcast = bc->n;
        kp.bcast_relu = bc->relu;
        for (int k = 0; k < bc->n; ++k) kp.bcast[k] = bc->dst[k];
    }
    kp.desc = p->d_desc;
    kp.col = p->d_col;
    kp.val = p->d_val;
    kp.x = x;
    kp.y = y;
    kp.ldx = ldx;
    kp.ldy = ldy;
    kp.f = f;
    kp.slab_w = c.sh.slab_w;
    kp.n_items = p->n_items;
    kp.n_prefix = p->n_prefix;
    kp.group = c.group;
    kp.n_pclaims = c.n_pclaims;
    kp.claims_per_slab = c.claims_per_slab;
    kp.n_claims = c.n_claims;
    kp.scratch = scratch;
    kp.n_partial = p->n_partial;
    kp.counter = counter;
    kp.flags = flags;
    kp.epoch = epoch;
    kp.status = p->d_status;
    kp.mode = mode;
    kp.use_scale = use_scale ? 1 : 0;
    kp.wait_ns = 2000000000ULL;
    if (c.tma) return launch_tma<256, 16, 2, 7>(kp, p->sm_count, s);
    if (c.sh.v4) {
        if (c.sh.nv == 1) return launch_regs<1, true>(kp, p->n_blocks, p->sm_count, s);
        if (c.sh.nv == 2) return launch_regs<2, true>(kp, p->n_blocks, p->sm_count, s);
        return launch_regs<4, true>(kp, p->n_blocks, p->sm_count, s);
    }
    if (c.sh.nv == 1) return launch_regs<1, false>(kp, p->n_blocks, p->sm_count, s);
    if (c.sh.nv == 2) return launch_regs<2, false>(kp, p->n_blocks, p->sm_count, s);
    return launch_regs<4, false>(kp, p->n_blocks, p->sm_count, s);
}

int run_plan(cbm_b200_plan* p, const char* who, const float* x, i64 ldx, float* y, i64 ldy, i32 f,
             int mode, bool use_scale, cudaStream_t s, const Bcast* bc = nullptr) {
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
    LaunchCfg c;
    rc = plan_cfg(p, who, x, ldx, y, ldy, f, mode, c);
    if (rc) return rc;

    if (c.need_flags > p->flags_cap) {
        // Growing the flag array: the old one may still be read by a launch in flight.
        CBM_CUDA(cudaStreamSynchronize(s));
        cudaFree(p->d_flags);
        p->d_flags = nullptr;
        p->device_bytes -= p->flags_cap * (i64)sizeof(i32);
        p->flags_cap = 0;
        CBM_CUDA(cudaMalloc((void**)&p->d_flags, (size_t)c.need_flags * sizeof(i32)));
        CBM_CUDA(cudaMemset(p->d_flags, 0, (size_t)c.need_flags * sizeof(i32)));
        p->flags_cap = c.need_flags;
        p->device_bytes += c.need_flags * (i64)sizeof(i32);
    }
    if (c.need_scratch > p->scratch_cap) {
        CBM_CUDA(cudaStreamSynchronize(s));
        cudaFree(p->d_scratch);
        p->d_scratch = nullptr;
        p->device_bytes -= p->scratch_cap * (i64)sizeof(float);
        p->scratch_cap = 0;
        CBM_CUDA(cudaMalloc((void**)&p->d_scratch, (size_t)c.need_scratch * sizeof(float)));
        p->scratch_cap = c.need_scratch;
        p->device_bytes += c.need_scratch * (i64)sizeof(float);
    }
    if (p->epoch == INT32_MAX) {  // epochs exhausted: start over on clean flags
        CBM_CUDA(cudaMemsetAsync(p->d_flags, 0, (size_t)p->flags_cap * sizeof(i32), s));
        p->epoch = 0;
    }
    return launch_plan(p, c, x, ldx, y, ldy, f, mode, use_scale, p->d_counter, p->d_flags, p->d_scratch,
                       ++p->epoch, s, bc);
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

extern "C" int cbm_b200_spmm_update_bcast(cbm_b200_plan* p, const float* x, int64_t ldx, float* y,
                                          int64_t ldy, int32_t f, int32_t normalized, int32_t relu,
                                          int32_t n_dst, float* const* dst, void* stream) {
    if (n_dst < 0 || n_dst > CBM_B200_MAX_BCAST || (n_dst > 0 && !dst))
        return cbm::fail(CBM_B200_ERR_ARG, "spmm_update_bcast: between 0 and " +
                                               std::to_string(CBM_B200_MAX_BCAST) + " destinations");
    Bcast bc;
    bc.n = n_dst;
    bc.relu = relu != 0;
    const bool v4 = (f % 4 == 0) && (ldy % 4 == 0);
    for (int k = 0; k < n_dst; ++k) {
        if (!dst[k]) return cbm::fail(CBM_B200_ERR_ARG, "spmm_update_bcast: NULL destination");
        if (dst[k] == x) return cbm::fail(CBM_B200_ERR_ARG, "spmm_update_bcast: a destination aliases x");
        if (v4 && aligned16(y) && !aligned16(dst[k]))
            return cbm::fail(CBM_B200_ERR_ARG, "spmm_update_bcast: destinations must be 16-byte aligned like y");
        bc.dst[k] = dst[k];
    }
    return run_plan(p, "spmm_update_bcast", x, ldx, y, ldy, f, MODE_FUSED, normalized != 0,
                    (cudaStream_t)stream, &bc);
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
    const Shape sh = pick_shape(f, 256, can_v4, 0);
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
    // The staging buffers use a leading dimension rounded up to 32 floats, so that rows start on
    // 128-byte lines whatever f is; chunks whose width is a multiple of 4 then take the 128-bit
    // path; a ragged last chunk is cut into a 128-bit part and a scalar tail of 1-3 columns.
    const i64 ld = ((i64)f + 31) / 32 * 32;  // whole 128-byte lines per row: gathered pieces fill whole lines
    const i64 xb = (i64)p->n_labels * ld, yb = (i64)p->n_out * ld;
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
    std::vector<std::pair<i32, i32>> chunks;  // (first column, width)
    for (i32 c0 = 0; c0 < f; c0 += chunk) {
        const i32 w = std::min(chunk, f - c0);
        if (w % 4 != 0 && w > 4) {  // ragged end: a 128-bit part and a short scalar tail
            chunks.emplace_back(c0, w / 4 * 4);
            chunks.emplace_back(c0 + w / 4 * 4, w % 4);
        } else {
            chunks.emplace_back(c0, w);
        }
    }
    const i32 n_chunks = (i32)chunks.size();
    if (!p->copy_in) CBM_CUDA(cudaStreamCreateWithFlags(&p->copy_in, cudaStreamNonBlocking));
    if (!p->copy_out) CBM_CUDA(cudaStreamCreateWithFlags(&p->copy_out, cudaStreamNonBlocking));
    while ((i32)p->events.size() < 2 * n_chunks) {
        cudaEvent_t e;
        CBM_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        p->events.push_back(e);
    }
    cudaStream_t s = p->own_stream;
    const size_t pitch = (size_t)f * sizeof(float), dpitch = (size_t)ld * sizeof(float);
    for (i32 k = 0; k < n_chunks; ++k) {
        const i32 c0 = chunks[k].first;
        const i32 w = chunks[k].second;
        CBM_CUDA(cudaMemcpy2DAsync(p->stage_x + c0, dpitch, x + c0, pitch, (size_t)w * sizeof(float),
                                       (size_t)p->n_labels, cudaMemcpyHostToDevice, p->copy_in));
        CBM_CUDA(cudaEventRecord(p->events[2 * k], p->copy_in));
        CBM_CUDA(cudaStreamWaitEvent(s, p->events[2 * k], 0));
        int rc = run_plan(p, "spmm_update_host", p->stage_x + c0, ld, p->stage_y + c0, ld, w, MODE_FUSED,
                          normalized != 0, s);
        if (rc) return rc;
        CBM_CUDA(cudaEventRecord(p->events[2 * k + 1], s));
        CBM_CUDA(cudaStreamWaitEvent(p->copy_out, p->events[2 * k + 1], 0));
        CBM_CUDA(cudaMemcpy2DAsync(y + c0, pitch, p->stage_y + c0, dpitch, (size_t)w * sizeof(float),
                                   (size_t)p->n_out, cudaMemcpyDeviceToHost, p->copy_out));
    }
    CBM_CUDA(cudaStreamSynchronize(p->copy_out));
    return cbm_b200_plan_status(p, s);
}

// Strided copy between host and device memory on a stream: one column chunk of a row-major operand
// (what the host-operand pipelines move).  A thin wrapper so that a host language without access to
// the CUDA runtime's 2-D copy can drive its own pipeline (cbm4gnn_b200/sharding.py does).
extern "C" int cbm_b200_copy2d_async(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch,
                                     int64_t width_bytes, int64_t rows, int32_t to_device, void* stream) {
    if (!dst || !src || width_bytes < 0 || rows < 0 || dst_pitch < width_bytes || src_pitch < width_bytes)
        return cbm::fail(CBM_B200_ERR_ARG, "copy2d_async: bad arguments");
    if (width_bytes == 0 || rows == 0) return CBM_B200_OK;
    CBM_CUDA(cudaMemcpy2DAsync(dst, (size_t)dst_pitch, src, (size_t)src_pitch, (size_t)width_bytes, (size_t)rows,
                               to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return CBM_B200_OK;
}

// ------------------------------------------------------------------------------------------
// Self-test of the bounded wait: one warp waits, with a limit of `wait_ms`, for a ready flag that
// nothing ever sets, and must come back with the timeout status instead of spinning forever.
// Exercises exactly the wait the product kernels use, without disturbing any plan.
// ------------------------------------------------------------------------------------------
namespace {
__global__ void wait_probe_kernel(i32* flag_and_status, u64 wait_ns) {
    const bool ok = wait_ready(flag_and_status, 1, flag_and_status + 1, wait_ns);
    if (threadIdx.x == 0) flag_and_status[2] = ok ? 1 : 0;
}
}  // namespace

extern "C" int cbm_b200_selftest_wait(int32_t device, int32_t wait_ms, void* stream) {
    if (wait_ms <= 0 || wait_ms > 1000)
        return cbm::fail(CBM_B200_ERR_ARG, "selftest_wait: wait_ms must be in 1..1000");
    DeviceGuard g(device);
    if (!g.ok) return cbm::fail(CBM_B200_ERR_CUDA, "selftest_wait: cudaSetDevice failed");
    i32* d = nullptr;
    CBM_CUDA(cudaMalloc((void**)&d, 3 * sizeof(i32)));
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(d, 0, 3 * sizeof(i32), s);
    i32 h[3] = {0, 0, -1};
    if (e == cudaSuccess) {
        wait_probe_kernel<<<1, 32, 0, s>>>(d, (u64)wait_ms * 1000000ULL);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(h, d, sizeof(h), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFree(d);
    if (e != cudaSuccess) return cbm::fail(CBM_B200_ERR_CUDA, std::string("selftest_wait: ") + cudaGetErrorString(e));
    if (h[1] == CBM_B200_ERR_TIMEOUT && h[2] == 0)
        return cbm::fail(CBM_B200_ERR_TIMEOUT, "selftest_wait: the wait ran out as it should");
    return cbm::fail(CBM_B200_ERR_FORMAT, "selftest_wait: the wait did not report a timeout");
}

// ------------------------------------------------------------------------------------------
// Measurement aid: the rate at which all SMs together stream a buffer that is resident in L2
// (32 MB, read 64 times with L2-only 128-bit loads, eight independent loads in flight per thread).
// The product kernels gather operand rows out of L2, so this rate — not the HBM rate — is the
// ceiling of their gather traffic; bench.py reports the gather rate against it.
// ------------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(512) l2_read_probe_kernel(const float4* __restrict__ buf, u64 n_vec, int rounds,
                                                            float* sink) {
    const u64 stride = (u64)gridDim.x * blockDim.x;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < rounds; ++r) {
        for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i + 7 * stride < n_vec; i += 8 * stride) {
            float4 t[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) t[k] = __ldcg(buf + i + (u64)k * stride);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                a.x += t[k].x;
                a.y += t[k].y;
                a.z += t[k].z;
                a.w += t[k].w;
            }
        }
    }
    if (a.x + a.y + a.z + a.w == 12345.678f) *sink = a.x;  // keeps the loads alive
}
}  // namespace

extern "C" double cbm_b200_probe_l2_read_gbps(int32_t device) {
    DeviceGuard g(device);
    if (!g.ok) return -1.0;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int threads = 512, blocks = sms * 2;
    const u64 per_pass = (u64)blocks * threads * 8;            // vectors read per sweep of the grid
    const u64 n_vec = ((32ull << 20) / 16) / per_pass * per_pass;  // about 32 MB, a whole number of sweeps
    float4* buf = nullptr;
    float* sink = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    double out = -1.0;
    if (cudaMalloc((void**)&buf, n_vec * 16) == cudaSuccess && cudaMalloc((void**)&sink, 4) == cudaSuccess &&
        cudaMemset(buf, 0, n_vec * 16) == cudaSuccess && cudaEventCreate(&e0) == cudaSuccess &&
        cudaEventCreate(&e1) == cudaSuccess) {
        const int rounds = 64;
        l2_read_probe_kernel<<<blocks, threads>>>(buf, n_vec, 4, sink);  // warm-up: brings the buffer into L2
        cudaEventRecord(e0);
        l2_read_probe_kernel<<<blocks, threads>>>(buf, n_vec, rounds, sink);
        cudaEventRecord(e1);
        float ms = 0.f;
        if (cudaEventSynchronize(e1) == cudaSuccess && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess && ms > 0.f)
            out = (double)n_vec * 16.0 * rounds / (ms * 1e-3) / 1e9;
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(buf);
    cudaFree(sink);
    return out;
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

    LaunchCfg c;
    rc = plan_cfg(p, who, x, ldx, y, ldy, f, MODE_FUSED, c);
    if (rc) return rc;
    // layout inside the fixed array: counters | ready flags | partial sums
    const i64 off_flags = 256;
    const i64 off_slots = off_flags + round_up_256(c.need_flags * (i64)sizeof(i32));
    const i64 need = off_slots + c.need_scratch * (i64)sizeof(float);
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
    CBM_CUDA(cudaMemsetAsync(base, 0, (size_t)(off_flags + c.need_flags * (i64)sizeof(i32)), s));
    // flags were just cleared, so any non-zero mark will do as this launch's epoch
    return launch_plan(p, c, x, ldx, y, ldy, f, MODE_FUSED, normalized != 0,
                       reinterpret_cast<u64*>(base), reinterpret_cast<i32*>(base + off_flags),
                       reinterpret_cast<float*>(base + off_slots), 1, s);
}
