/*
 * cbm_b200.h — C ABI of libcbm_b200.so: the compressed-binary-matrix (CBM) product engine for
 * NVIDIA B200 (sm_100a).
 *
 * The library replaces, for the CBM product path only, the pybind11 module `cbm.cbm_mkl_cpp` of
 * cbm4scale/cbm4gnn (cbm/cbm_extensions.cpp:1757-1771).  Every entry point takes plain pointers
 * and sizes, returns an `int` status (0 = success) and leaves a message retrievable with
 * cbm_b200_last_error() on failure.  Nothing here calls exit(); nothing here takes a torch type.
 *
 * Conventions shared with the reference: int32 indices, fp32 values, dense operands row-major.
 * A "tree" is the reference's (mst_row[n+2], mst_col[n]) CSR over n+1 vertices whose last vertex n
 * is the virtual all-zero root (cbm/cbm_extensions.cpp:274-286); "deltas" is the n x n CSR of
 * signed differences between each row and its tree parent (cbm/cbm_extensions.cpp:186-261).
 *
 * Device pointers are marked [dev], host pointers [host].  `stream` is a cudaStream_t passed as
 * void* (NULL = the legacy default stream).  Launches are asynchronous on that stream.
 */
#ifndef CBM_B200_H
#define CBM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define CBM_B200_OK 0
#define CBM_B200_ERR_ARG 1      /* bad argument (null pointer, size, dtype contract, aliasing) */
#define CBM_B200_ERR_CUDA 2     /* a CUDA runtime call failed */
#define CBM_B200_ERR_FORMAT 3   /* tree / delta arrays are not a valid CBM structure */
#define CBM_B200_ERR_TIMEOUT 4  /* a bounded device-side wait ran out (reported by *_status) */
#define CBM_B200_ERR_ALLOC 5    /* host or device allocation failed */

typedef struct cbm_b200_built cbm_b200_built; /* result of the host builder (host memory only)   */
typedef struct cbm_b200_plan cbm_b200_plan;   /* device-resident schedule for one GPU            */

/* Message of the last failure on the calling thread ("" if none). */
const char* cbm_b200_last_error(void);

/* Library / build identification: returns e.g. "cbm_b200 0.1 sm_100a". */
const char* cbm_b200_version(void);

/* --------------------------------------------------------------------------------------------
 * Host builder.  Replaces cbm_init_v1_ (cbm/cbm_extensions.cpp:8-326, col_mul == NULL) and
 * cbm_init_v2_ (cbm/cbm_extensions.cpp:328-644, col_mul != NULL), bound in the reference as
 * from_coo_int32_t_v1_ / from_coo_int32_t_v2_ (cbm/cbm_extensions.cpp:1758-1759).
 *
 * Input: a coalesced COO pattern (row[i], col[i]) of an n x n binary matrix [host].  Values are
 * not needed (the reference passes all-ones only because MKL's syrk wants them).
 * Candidate rule, virtual edges and weights follow cbm/cbm_extensions.cpp:75-102:
 *   h(r,c) = |r| + |c| - 2|r ∩ c|;  edge c->r iff h < |r| - alpha;  edge r->c iff h < |c| - alpha;
 *   edge root->r with weight |r| for every r.
 * The minimum-cost arborescence rooted at vertex n is computed by the library's own solver (the
 * reference delegates to the external arbok::TarjanPQ, cbm/cbm_extensions.cpp:109-148).  Ties are
 * broken deterministically (lowest adjusted weight, then lowest source id), so the same input
 * always yields byte-identical output.
 * n_threads <= 0 uses every hardware thread.
 * ------------------------------------------------------------------------------------------ */
int cbm_b200_build(const int32_t* row, const int32_t* col, int64_t nnz, int32_t n, int32_t alpha,
                   const float* col_mul, int32_t n_threads, cbm_b200_built** out);

/* The same builder with its candidate search — over 95 % of the build on high-degree graphs — on
 * CUDA device `device` (one thread block per possible parent row, hit counters in L2); arborescence
 * and deltas stay on the host.  The candidate set, hence the structure, is identical to
 * cbm_b200_build's.  Falls back to the host search when the GPU cannot be used (no device, out of
 * memory); cbm_b200_built_candidates_on_gpu tells which ran (1 = GPU). */
int cbm_b200_build_gpu(const int32_t* row, const int32_t* col, int64_t nnz, int32_t n, int32_t alpha,
                       const float* col_mul, int32_t n_threads, int32_t device, cbm_b200_built** out);
int cbm_b200_built_candidates_on_gpu(const cbm_b200_built* b);

/* Sizes and statistics of a built structure.  Any out-pointer may be NULL.
 *   n_delta       number of delta entries (= total weight of the arborescence)
 *   n_candidates  number of candidate edges offered to the solver, virtual edges included
 *   n_root_children, depth   shape of the tree (depth of a root child = 1)
 *   seconds[4]    wall time of: CSR + candidate graph, arborescence, delta emission, total */
int cbm_b200_built_info(const cbm_b200_built* b, int64_t* n_delta, int64_t* n_candidates,
                        int32_t* n_root_children, int32_t* depth, double* seconds);

/* Copy the structure out [host].  mst_row has n+2 entries, mst_col n (children sorted by id).
 * delta_crow has n+1 entries; delta_col / delta_val have n_delta, columns ascending inside a row:
 * the CSR the reference obtains by coalescing its COO output (cbm/cbm.py:120-141).  parent (n
 * entries, the virtual root written as n) may be NULL. */
int cbm_b200_built_export_csr(const cbm_b200_built* b, int32_t* mst_row, int32_t* mst_col,
                              int32_t* delta_crow, int32_t* delta_col, float* delta_val,
                              int32_t* parent);

/* The same deltas in the reference's native output layout: COO triples in breadth-first order of
 * the tree (cbm/cbm_extensions.cpp:166-270, 288-325).  Each array has n_delta entries. */
int cbm_b200_built_export_coo(const cbm_b200_built* b, int32_t* delta_row, int32_t* delta_col,
                              float* delta_val);

void cbm_b200_built_free(cbm_b200_built* b);

/* --------------------------------------------------------------------------------------------
 * Plans.  A plan is the device-side schedule derived from the reference-format arrays; the arrays
 * themselves are consumed unmodified.  It plays the role of the MKL handle the reference re-creates
 * on every call (cbm/cbm_extensions.cpp:679, 1134, 1252) plus the DFS stack of its tree walk.
 *
 * All array arguments are [host].  `multiplier` (n floats, D^-1/2) may be NULL for the
 * unnormalized product.  Sharding: `perm` (n entries, NULL = identity) relabels vertices with
 * distinct labels in [0, n_labels), n_labels >= n (n_labels = 0 means n; labels that no vertex
 * carries are padding that lets every shard have the same number of rows).  The plan computes only
 * rows whose label lies in [own_begin, own_end); those rows must form whole subtrees of the
 * virtual root.  In every product call the dense right-hand side is indexed by LABEL (n_labels
 * rows), and the output pointer addresses the shard: output row (label - own_begin); padding rows
 * of the output are never written.  own_begin = 0, own_end = n_labels computes everything.
 * `device` is the CUDA device ordinal that owns the plan.
 * ------------------------------------------------------------------------------------------ */
int cbm_b200_plan_create(int32_t n, const int32_t* mst_row, const int32_t* mst_col,
                         const int32_t* delta_crow, const int32_t* delta_col,
                         const float* delta_val, const float* multiplier, const int32_t* perm,
                         int32_t n_labels, int32_t own_begin, int32_t own_end, int32_t device,
                         cbm_b200_plan** out);

void cbm_b200_plan_destroy(cbm_b200_plan* p);

/* Host-only twin of cbm_b200_plan_create (same arguments minus the device): builds the schedule,
 * runs the pre-launch checks (every item waits only for earlier items, whoever is waited for
 * publishes, every row produced and every parked partial sum collected exactly once) and reports
 * its sizes.  Needs no GPU; plan_create runs the same checks. */
int cbm_b200_schedule_info(int32_t n, const int32_t* mst_row, const int32_t* mst_col,
                           const int32_t* delta_crow, const int32_t* delta_col,
                           const float* delta_val, const float* multiplier, const int32_t* perm,
                           int32_t n_labels, int32_t own_begin, int32_t own_end, int32_t* n_items,
                           int32_t* n_prefix, int32_t* n_partial, int32_t* n_rows);

/* Figures used by the byte model: rows computed by this plan, delta entries of those rows, rows
 * whose parent is the virtual root, tree depth, and device bytes held by the plan. */
int cbm_b200_plan_info(const cbm_b200_plan* p, int32_t* n_rows, int64_t* n_delta,
                       int32_t* n_root_children, int32_t* depth, int64_t* device_bytes);

/* Tuning knobs (0 keeps the default): column-slab width in floats, thread blocks per launch, the
 * column-chunk width (a multiple of 4) of the host-buffer pipeline below, and the kernel form
 * (0 = gather held in registers, the default; 1 = operand rows staged in shared memory by bulk
 * asynchronous copies, for 16-byte aligned operands whose width is a multiple of 4). */
int cbm_b200_plan_tune(cbm_b200_plan* p, int32_t slab_width, int32_t n_blocks, int32_t host_chunk,
                       int32_t form);

/* Waits for `stream`, then reports whether any launch since the last call gave up on a bounded
 * wait (CBM_B200_ERR_TIMEOUT) — in that case the outputs of that launch are invalid. */
int cbm_b200_plan_status(cbm_b200_plan* p, void* stream);

/* --------------------------------------------------------------------------------------------
 * Products.  x [dev]: n_labels x f floats with leading dimension ldx; y [dev]:
 * (own_end-own_begin) x f with leading dimension ldy; x and y must not overlap.
 *
 * cbm_b200_spmm_update        y = A x: delta product fused with the tree update y_v += y_parent.
 *                             Replaces seq_/omp_s_spmm_update_csr_int32
 *                             (cbm/cbm_extensions.cpp:650-740, 1108-1219).
 * cbm_b200_fused_spmm_update  y = D^-1/2 A D^-1/2 x for a plan created with `multiplier`:
 *                             y_r *= s_r for root children, y_v = (y_v + y_u / s_u) s_v below.
 *                             Replaces seq_/omp_s_fused_spmm_update_csr_int32
 *                             (cbm/cbm_extensions.cpp:845-996, 1224-1374).
 * cbm_b200_update             in-place tree update of y that already holds the delta product.
 *                             Replaces seq_/omp_s_update_csr_int32 and omp_s_update_avx_int32
 *                             (cbm/cbm_extensions.cpp:742-786, 1485-1610, 1612-1705).
 * cbm_b200_fused_update       normalized in-place update.  Replaces seq_/omp_s_fused_update_csr_int32
 *                             (cbm/cbm_extensions.cpp:998-1105, 1376-1483).
 * cbm_b200_delta_spmm         y = deltas x from the plan's resident copy of the delta CSR (the
 *                             `self.deltas @ x` step of cbm/cbm.py:255-275).
 * ------------------------------------------------------------------------------------------ */
int cbm_b200_spmm_update(cbm_b200_plan* p, const float* x, int64_t ldx, float* y, int64_t ldy,
                         int32_t f, void* stream);
int cbm_b200_fused_spmm_update(cbm_b200_plan* p, const float* x, int64_t ldx, float* y,
                               int64_t ldy, int32_t f, void* stream);
int cbm_b200_update(cbm_b200_plan* p, float* y, int64_t ldy, int32_t f, void* stream);
int cbm_b200_fused_update(cbm_b200_plan* p, float* y, int64_t ldy, int32_t f, void* stream);
int cbm_b200_delta_spmm(cbm_b200_plan* p, const float* x, int64_t ldx, float* y, int64_t ldy,
                        int32_t f, void* stream);

/* Plain CSR product y = M x for any fp32 CSR with device-resident arrays [dev].  Replaces
 * seq_/omp_s_spmm_csr_int32 (cbm/cbm_extensions.cpp:790-843, 1707-1755).  row_b / row_e are the
 * reference's 4-array form (row_b = crow[:-1], row_e = crow[1:]). */
int cbm_b200_csr_spmm(int32_t n_rows, const int32_t* row_b, const int32_t* row_e,
                      const int32_t* col, const float* val, const float* x, int64_t ldx, float* y,
                      int64_t ldy, int32_t f, void* stream);

/* The same product from a reusable plan: the counterpart of the oneMKL handle the reference
 * creates from these arrays before every product (mkl_sparse_s_create_csr,
 * cbm/cbm_extensions.cpp:1726-1734).  crow (n_rows + 1 entries), col, val are [host]; the plan
 * keeps its own device copy.  Long rows are cut into segments and balanced over the GPU like the
 * rows of a CBM structure, which the array form above (one warp per whole row) does not do.
 * y = M x is then cbm_b200_spmm_update(plan, x, ...) with x of n_cols rows and y of n_rows rows. */
int cbm_b200_csr_plan_create(int32_t n_rows, int32_t n_cols, const int32_t* crow, const int32_t* col,
                             const float* val, int32_t device, cbm_b200_plan** out);

/* Multi-GPU form of the two fused products (no counterpart in the reference, which has no
 * distributed code): every finished row is written to y as usual and, after an optional ReLU,
 * to n_dst further buffers dst[k] [dev, possibly memory of a peer GPU mapped into this process]
 * with y's layout and leading dimension — the place this shard occupies in each GPU's copy of
 * the gathered layer output.  The stores to peers are ordinary stores issued by the product
 * kernel as rows finish, so the exchange overlaps the product; the caller synchronises the GPUs
 * afterwards.  y always receives the rows without the ReLU (children in the tree read them).
 * At most CBM_B200_MAX_BCAST destinations. */
#define CBM_B200_MAX_BCAST 8
int cbm_b200_spmm_update_bcast(cbm_b200_plan* p, const float* x, int64_t ldx, float* y, int64_t ldy,
                               int32_t f, int32_t normalized, int32_t relu, int32_t n_dst,
                               float* const* dst, void* stream);

/* Host-buffer forms of the two fused products: x [host] n_labels x f and y [host]
 * (own_end-own_begin) x f, both contiguous (ld = f).  The call copies x to the device, runs the product and copies y back on the
 * plan's own stream, and returns when y is complete.  Staging buffers belong to the plan and grow
 * on demand.  `normalized` != 0 selects cbm_b200_fused_spmm_update.  These are what a caller
 * holding CPU tensors, as every caller of the reference does, binds to. */
int cbm_b200_spmm_update_host(cbm_b200_plan* p, const float* x, float* y, int32_t f,
                              int32_t normalized);

/* Strided (2-D) copy of `rows` pieces of `width_bytes` between host and device memory on `stream`
 * (to_device != 0: host -> device): one column chunk of a row-major operand.  No counterpart in the
 * reference; lets a host-side pipeline over column chunks (multi-GPU host-operand product) be
 * written without binding the CUDA runtime. */
int cbm_b200_copy2d_async(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch,
                          int64_t width_bytes, int64_t rows, int32_t to_device, void* stream);

/* Self-test of the device-side bounded wait (the reference has no counterpart: its CPU walk cannot
 * stall).  One warp waits at most wait_ms (1..1000) for a flag that is never set; the call returns
 * CBM_B200_ERR_TIMEOUT when the wait gave up as designed, any other status is a failure.  The
 * context stays usable. */
int cbm_b200_selftest_wait(int32_t device, int32_t wait_ms, void* stream);

/* --------------------------------------------------------------------------------------------
 * Dense maps of the GCN layers: `lin` of gnns/graph_convolutional_network/cbm_gcn.py:21-24 (a
 * bias-free [N,in] x [in,out] fp32 map, there torch_geometric's Linear on the CPU) and its two
 * gradients, as fp32-accurate GEMMs on the tensor cores (every operand split into three bf16
 * terms, fp32 accumulation in tensor memory).  All pointers [dev], row-major, 16-byte aligned;
 * n_in, n_out and every leading dimension must be multiples of 4 floats.
 *   cbm_b200_dense_forward      y [n_rows,n_out] = x [n_rows,n_in] * w^T,  w [n_out,n_in]
 *   cbm_b200_dense_forward_relu y = max(x * w^T, 0): the map followed by the ReLU that sits between two
 *                               layers (benchmark/parallel/benchmark_gcn_cpu.py:70-89), in the epilogue
 *   cbm_b200_dense_grad_input   dx [n_rows,n_in] = dy [n_rows,n_out] * w
 *   cbm_b200_dense_grad_input_relu  the same, set to 0 wherever h [n_rows,n_in] is 0: the gradient that
 *                               flows back through the ReLU whose output h was (the mask in the epilogue)
 *   cbm_b200_dense_grad_weight  dw [n_out,n_in]  = dy^T * x; contracts over the rows in up to
 *                               CBM_B200_DENSE_MAX_CHUNKS independent chunks whose partial results
 *                               are summed in a fixed order; `workspace` [dev] must hold
 *                               cbm_b200_dense_grad_weight_workspace(...) bytes.
 * ------------------------------------------------------------------------------------------ */
#define CBM_B200_DENSE_MAX_CHUNKS 296
int cbm_b200_dense_forward(const float* x, int64_t ldx, const float* w, int64_t ldw, float* y,
                           int64_t ldy, int32_t n_rows, int32_t n_in, int32_t n_out, void* stream);
int cbm_b200_dense_forward_relu(const float* x, int64_t ldx, const float* w, int64_t ldw, float* y,
                                int64_t ldy, int32_t n_rows, int32_t n_in, int32_t n_out, void* stream);
int cbm_b200_dense_grad_input(const float* dy, int64_t lddy, const float* w, int64_t ldw, float* dx,
                              int64_t lddx, int32_t n_rows, int32_t n_in, int32_t n_out, void* stream);
int cbm_b200_dense_grad_input_relu(const float* dy, int64_t lddy, const float* w, int64_t ldw, const float* h,
                                   int64_t ldh, float* dx, int64_t lddx, int32_t n_rows, int32_t n_in,
                                   int32_t n_out, void* stream);
int64_t cbm_b200_dense_grad_weight_workspace(int32_t n_rows, int32_t n_in, int32_t n_out);
int cbm_b200_dense_grad_weight(const float* dy, int64_t lddy, const float* x, int64_t ldx, float* dw,
                               int64_t lddw, int32_t n_rows, int32_t n_in, int32_t n_out,
                               void* workspace, int64_t workspace_bytes, void* stream);

/* Measurement aid (no counterpart in the reference): GB/s at which all SMs of `device` together
 * stream a 32 MB buffer that stays resident in L2 — the ceiling of the gather traffic of the
 * product kernels.  Allocates and frees its buffer; returns a negative number on failure. */
double cbm_b200_probe_l2_read_gbps(int32_t device);

/* --------------------------------------------------------------------------------------------
 * The fused product for callers that must not allocate.  (No counterpart in the reference, whose
 * CPU kernels need no scratch memory; added for GPU callers.)
 *
 * Who needs it: a caller that cannot reach cudaMalloc once it is running — it gave all device
 * memory to its own pool, it runs while a stream is being captured, or it cannot afford the
 * device-wide synchronisation an allocation implies.  The entry points above allocate their
 * ready-flag and partial-sum buffers on demand; this one performs the same product (same kernel,
 * same results) with that scratch taken from a fixed array of CBM_B200_STATIC_SCRATCH_BYTES that
 * is part of the library image, so every GPU that loads the library holds that much memory until
 * the process exits.  The call itself allocates and frees nothing.
 *
 * `normalized` != 0 computes what cbm_b200_fused_spmm_update computes, 0 what cbm_b200_spmm_update
 * computes.  x, y, ldx, ldy, f, stream as there.  A product whose scratch need (4 bytes per row
 * segment and column slab, plus the partial sums of rows longer than 192 delta entries) exceeds
 * the fixed array is refused with CBM_B200_ERR_ARG and a message giving both sizes.
 *
 * The first call on each device looks up the array's device address; make that first call before
 * any stream capture begins.  All calls on a device share the array and each call clears the part
 * it uses, so two of these calls that overlap on one GPU (different streams or threads) race:
 * the caller must order them.  Timeouts are reported through cbm_b200_plan_status as usual.
 * ------------------------------------------------------------------------------------------ */
#define CBM_B200_STATIC_SCRATCH_BYTES (8u << 20)
int cbm_b200_spmm_update_static(cbm_b200_plan* p, const float* x, int64_t ldx, float* y,
                                int64_t ldy, int32_t f, int32_t normalized, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CBM_B200_H */
