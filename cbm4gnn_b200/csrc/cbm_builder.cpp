// Host builder of the CBM structure: candidate graph, minimum-cost arborescence, deltas.
//
// Restates, with its own data structures, what cbm_init_v1_ / cbm_init_v2_ do in the reference
// (cbm/cbm_extensions.cpp:8-326 and 328-644):
//   1. pattern -> CSR (the reference uses MKL's COO->CSR conversion, :15-43);
//   2. row-pair intersection counts (the reference materialises A*A^T with mkl_sparse_syrk, :47;
//      here the counts are produced row block by row block and filtered on the fly, so the
//      product is never stored);
//   3. candidate edges with the reference's rule (:75-102);
//   4. minimum-cost arborescence rooted at the virtual vertex n (the reference calls the external
//      arbok::TarjanPQ, :109-148; this file has its own contraction/expansion solver);
//   5. breadth-first traversal, sorted-merge deltas and the tree CSR (:150-286).
// Everything runs on the host; the GPU engine consumes the arrays this file emits unmodified.

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <memory>
#include <vector>

#include <omp.h>

#include "cbm_b200.h"
#include "cbm_candidates.h"
#include "cbm_common.h"

namespace {

using i32 = int32_t;
using i64 = int64_t;

double now_s() {
    using clk = std::chrono::steady_clock;
    return std::chrono::duration<double>(clk::now().time_since_epoch()).count();
}

// ------------------------------------------------------------------------------------------
// Pattern CSR with sorted, de-duplicated columns.
// ------------------------------------------------------------------------------------------
struct Pattern {
    i32 n = 0;
    std::vector<i64> ptr;  // n+1
    std::vector<i32> idx;  // nnz
    i32 len(i32 r) const { return (i32)(ptr[r + 1] - ptr[r]); }
};

Pattern make_csr(const i32* row, const i32* col, i64 nnz, i32 n) {
    Pattern p;
    p.n = n;
    p.ptr.assign((size_t)n + 1, 0);
    for (i64 i = 0; i < nnz; ++i) p.ptr[(size_t)row[i] + 1]++;
    for (i32 r = 0; r < n; ++r) p.ptr[r + 1] += p.ptr[r];
    std::vector<i32> tmp((size_t)nnz);
    {
        std::vector<i64> cur(p.ptr.begin(), p.ptr.end() - 1);
        for (i64 i = 0; i < nnz; ++i) tmp[(size_t)cur[row[i]]++] = col[i];
    }
    // sort + dedupe each row, then compact
    std::vector<i32> newlen((size_t)n);
#pragma omp parallel for schedule(dynamic, 256)
    for (i32 r = 0; r < n; ++r) {
        i32* b = tmp.data() + p.ptr[r];
        i32* e = tmp.data() + p.ptr[r + 1];
        if (!std::is_sorted(b, e)) std::sort(b, e);
        newlen[r] = (i32)(std::unique(b, e) - b);
    }
    std::vector<i64> nptr((size_t)n + 1, 0);
    for (i32 r = 0; r < n; ++r) nptr[r + 1] = nptr[r] + newlen[r];
    p.idx.resize((size_t)nptr[n]);
#pragma omp parallel for schedule(static)
    for (i32 r = 0; r < n; ++r)
        std::copy(tmp.data() + p.ptr[r], tmp.data() + p.ptr[r] + newlen[r], p.idx.data() + nptr[r]);
    p.ptr.swap(nptr);
    return p;
}

Pattern transpose(const Pattern& a) {
    Pattern t;
    t.n = a.n;
    t.ptr.assign((size_t)a.n + 1, 0);
    for (i32 c : a.idx) t.ptr[(size_t)c + 1]++;
    for (i32 r = 0; r < a.n; ++r) t.ptr[r + 1] += t.ptr[r];
    t.idx.resize(a.idx.size());
    std::vector<i64> cur(t.ptr.begin(), t.ptr.end() - 1);
    for (i32 r = 0; r < a.n; ++r)
        for (i64 k = a.ptr[r]; k < a.ptr[r + 1]; ++k) t.idx[(size_t)cur[a.idx[k]]++] = r;
    return t;  // rows inside each column list come out ascending
}

// ------------------------------------------------------------------------------------------
// Candidate graph.  An in-edge of vertex `dst`: (src, weight).
// ------------------------------------------------------------------------------------------
struct InEdge {
    i32 src;
    i32 w;
};

struct Candidates {
    std::vector<i64> off;     // n+1: in-edges of v are e[off[v] .. off[v+1])
    std::vector<InEdge> e;    // first entry of every list is the virtual edge (n -> v, |v|)
    i64 total = 0;
};

// The reference tests every pair of rows that share a column (the non-zeros of A*A^T,
// cbm/cbm_extensions.cpp:87-102).  The same set of candidate edges is produced here without
// visiting all those pairs: an edge u -> v passes the rule  h(u,v) < |v| - alpha  exactly when
// |u ∩ v| > (|u| + alpha) / 2, i.e. when at least t = floor((|u| + alpha) / 2) + 1 of u's columns
// are also in v.  Order all columns from rarest to most frequent.  If u and v share t columns,
// then for any j <= t at least j of them lie among u's first |u| - t + j columns in that order
// (only t - j columns lie behind them).  So for every possible parent u the rows holding its rare
// columns are counted through the column lists — hub columns, which make A*A^T explode, almost
// never fall in that prefix — and only rows reaching j hits get their intersection with u counted
// exactly.
// device >= 0 runs the search on that GPU (cbm_candidates.cu) and falls back to the host when the
// GPU cannot be used; the result is the same set of edges either way.  *used_gpu reports which ran.
Candidates make_candidates(const Pattern& a, const Pattern& at, i32 alpha, int device = -1, bool* used_gpu = nullptr) {
    const i32 n = a.n;
    if (used_gpu) *used_gpu = false;
    struct Tri {
        i32 src, dst, w;
    };
    // rank of every column in the rare-to-frequent order (ties by id)
    std::vector<i32> by_freq((size_t)n);
    for (i32 c = 0; c < n; ++c) by_freq[c] = c;
    std::sort(by_freq.begin(), by_freq.end(), [&](i32 x, i32 y) {
        const i32 fx = at.len(x), fy = at.len(y);
        return fx != fy ? fx < fy : x < y;
    });
    std::vector<i32> rank((size_t)n);
    for (i32 i = 0; i < n; ++i) rank[by_freq[i]] = i;

    const i32 block = 64;
    const i32 n_blocks = (n + block - 1) / block;
    std::vector<std::vector<Tri>> found((size_t)n_blocks);
    std::vector<char> on_host;  // empty: every parent row is searched on the host

    if (device >= 0 && n > 0) {
        const bool trace = std::getenv("CBM_B200_BUILD_TRACE") != nullptr;
        const double t_a = now_s();
        // rows with their columns replaced by ranks, rarest first: a prefix of such a row is the
        // set of its rarest columns
        std::vector<i32> row_rank(a.idx.size());
#pragma omp parallel for schedule(dynamic, 256)
        for (i32 r = 0; r < n; ++r) {
            i32* b = row_rank.data() + a.ptr[r];
            for (i64 k = a.ptr[r]; k < a.ptr[r + 1]; ++k) row_rank[(size_t)k] = rank[a.idx[(size_t)k]];
            std::sort(b, b + a.len(r));
        }
        std::vector<cbm::CandTriple> triples;
        std::vector<i32> left;
        std::string err;
        const double t_b = now_s();
        if (trace) std::fprintf(stderr, "[cbm build] rank rows %.3f s\n", t_b - t_a);
        if (cbm::gpu_candidates(device, n, alpha, a.ptr.data(), row_rank.data(), by_freq.data(), at.ptr.data(),
                                at.idx.data(), triples, left, err) == 0) {
            if (used_gpu) *used_gpu = true;
            if (trace) std::fprintf(stderr, "[cbm build] gpu search %.3f s, %zu edges, %zu parents left to the host\n",
                                    now_s() - t_b, triples.size(), left.size());
            on_host.assign((size_t)n, 0);
            for (i32 u : left) on_host[u] = 1;
            // in the order the host search emits: by parent block, inside a block by (parent, child)
            for (const cbm::CandTriple& t : triples) found[(size_t)(t.src / block)].push_back({t.src, t.dst, t.w});
#pragma omp parallel for schedule(dynamic, 16)
            for (i32 b = 0; b < n_blocks; ++b)
                std::sort(found[b].begin(), found[b].end(),
                          [](const Tri& x, const Tri& y) { return x.src != y.src ? x.src < y.src : x.dst < y.dst; });
        }
    }
    std::vector<i32>().swap(by_freq);
    const bool host_all = on_host.empty();

#pragma omp parallel
    {
        std::vector<uint64_t> in_u(((size_t)n + 63) / 64, 0);  // bit per column: is it in row u?
                                                                // (16 KB at n = 132 534: stays in L1)
        // row -> shared columns seen inside u's prefix.  The counters are hit in random order once
        // per entry of every column list of the prefix, which is what the search spends its time
        // on, so they are kept 16 bits wide (265 KB at n = 132 534: stays in the core's L2); the
        // rare row whose prefix is longer than a 16-bit count can hold uses the 32-bit array.
        std::vector<uint16_t> hits16((size_t)n, 0);
        std::vector<i32> hits32;
        std::vector<i32> touched, cols;
#pragma omp for schedule(dynamic, 1)
        for (i32 b = 0; b < n_blocks; ++b) {
            std::vector<Tri>& out = found[b];
            const i32 u_end = std::min(n, (b + 1) * block);
            for (i32 u = b * block; u < u_end; ++u) {
                if (!host_all && !on_host[u]) continue;  // done on the GPU
                const i32 nu = a.len(u);
                // shared columns an edge u -> v needs: the smallest integer above (|u| + alpha) / 2,
                // and at least one (the reference only sees pairs that intersect)
                const i64 sum = (i64)nu + alpha;
                const i64 half_floor = sum >= 0 ? sum / 2 : -((-sum + 1) / 2);
                const i64 need64 = std::max<i64>(half_floor + 1, 1);
                if (need64 > nu) continue;  // no row can contain that many of u's columns
                const i32 need = (i32)need64;
                // hits demanded inside the prefix: more hits = longer prefix to count through but
                // fewer rows left for the exact intersection; need/8 within [8, 32] measured best
                const i32 j_hits = std::min(need, std::max(8, std::min(32, need / 8)));
                const i32 plen = nu - need + j_hits;
                const i32* ub = a.idx.data() + a.ptr[u];
                const i32* ue = a.idx.data() + a.ptr[u + 1];
                cols.assign(ub, ue);
                if (plen < nu)
                    std::partial_sort(cols.begin(), cols.begin() + plen, cols.end(),
                                      [&](i32 x, i32 y) { return rank[x] < rank[y]; });
                touched.clear();
                const bool wide = plen > 65000;
                if (wide && hits32.empty()) hits32.assign((size_t)n, 0);
                auto count_prefix = [&](auto& hits) {
                    for (i32 i = 0; i < plen; ++i) {
                        const i32 colk = cols[i];
                        for (i64 q = at.ptr[colk]; q < at.ptr[colk + 1]; ++q) {
                            const i32 v = at.idx[q];
                            if (hits[v]++ == 0) touched.push_back(v);
                        }
                    }
                };
                if (wide) count_prefix(hits32);
                else count_prefix(hits16);
                bool marked = false;
                const size_t out_before = out.size();
                for (i32 v : touched) {
                    const i32 in_prefix = wide ? hits32[v] : (i32)hits16[v];
                    if (wide) hits32[v] = 0;
                    else hits16[v] = 0;
                    if (v == u || in_prefix < j_hits) continue;
                    const i32 nv = a.len(v);
                    if (nv < need) continue;
                    i32 both = in_prefix;
                    if (plen < nu) {  // the frequent tail of u still has to be looked at
                        const i32* vb = a.idx.data() + a.ptr[v];
                        const i32* ve = a.idx.data() + a.ptr[v + 1];
                        if ((i64)nv <= (i64)12 * (nu - plen)) {
                            if (!marked) {
                                for (const i32* k = ub; k != ue; ++k) in_u[(size_t)*k >> 6] |= 1ull << (*k & 63);
                                marked = true;
                            }
                            both = 0;
                            for (const i32* k = vb; k != ve; ++k) both += (i32)((in_u[(size_t)*k >> 6] >> (*k & 63)) & 1ull);
                        } else {
                            for (i32 i = plen; i < nu; ++i) both += std::binary_search(vb, ve, cols[i]);
                        }
                    }
                    const i32 h = nu + nv - 2 * both;
                    if (h < nv - alpha) out.push_back({u, v, h});  // cbm/cbm_extensions.cpp:93-101
                }
                if (marked)
                    for (const i32* k = ub; k != ue; ++k) in_u[(size_t)*k >> 6] = 0;
                // only the few survivors are put in order (by child id); sorting every touched
                // row first was the most expensive step of the whole search
                std::sort(out.begin() + out_before, out.end(),
                          [](const Tri& x, const Tri& y) { return x.dst < y.dst; });
            }
        }
    }

    if (!host_all) {  // parents finished on the host were appended behind the GPU's: restore (parent, child) order
#pragma omp parallel for schedule(dynamic, 16)
        for (i32 b = 0; b < n_blocks; ++b)
            std::sort(found[b].begin(), found[b].end(),
                      [](const Tri& x, const Tri& y) { return x.src != y.src ? x.src < y.src : x.dst < y.dst; });
    }
    Candidates g;
    g.off.assign((size_t)n + 1, 0);
    for (i32 v = 0; v < n; ++v) g.off[v + 1] = 1;  // virtual edge
    for (auto& blk : found)
        for (const Tri& t : blk) g.off[(size_t)t.dst + 1]++;
    for (i32 v = 0; v < n; ++v) g.off[v + 1] += g.off[v];
    g.total = g.off[n];
    g.e.resize((size_t)g.total);
    std::vector<i64> cur(g.off.begin(), g.off.end() - 1);
    for (i32 v = 0; v < n; ++v) g.e[(size_t)cur[v]++] = {n, a.len(v)};
    for (auto& blk : found) {
        for (const Tri& t : blk) g.e[(size_t)cur[t.dst]++] = {t.src, t.w};
        std::vector<Tri>().swap(blk);
    }
    return g;
}

// ------------------------------------------------------------------------------------------
// Minimum-cost arborescence rooted at vertex n over the candidate graph.
//
// Contraction phase (Chu-Liu/Edmonds in the path-growing form of Tarjan 1977): grow a path of
// components, each choosing its cheapest in-edge from outside itself; a path that bites its own
// tail is contracted, in-edge queues are merged small-into-large with lazy offsets carrying the
// reduced costs.  Every choice becomes a node of a forest; the choices made by the members of a
// contracted cycle become children of the choice later made by the contracted component.
// Expansion phase (Camerini, Fratta, Maffioli 1979): repeatedly take a forest root, accept its
// edge, and dissolve the forest path from the leaf of the edge's head up to that root; the
// subtrees hanging off the path become new roots.
// ------------------------------------------------------------------------------------------
struct QEnt {
    i64 key;  // stored key; reduced cost = key + lazy[component]
    i32 src;
    i32 dst;
};
struct QCmp {  // std heap functions build a max-heap: invert for (key, src, dst) ascending
    bool operator()(const QEnt& x, const QEnt& y) const {
        if (x.key != y.key) return x.key > y.key;
        if (x.src != y.src) return x.src > y.src;
        return x.dst > y.dst;
    }
};

struct Arborescence {
    std::vector<i32> parent;  // n entries, virtual root written as n
};

bool solve_arborescence(const Candidates& g, i32 n, Arborescence& out, std::string& err) {
    const i32 V = n + 1;
    std::vector<i32> uf((size_t)V), uf_size((size_t)V, 1);
    for (i32 v = 0; v < V; ++v) uf[v] = v;
    auto find = [&](i32 v) {
        i32 r = v;
        while (uf[r] != r) r = uf[r];
        while (uf[v] != r) {
            i32 nx = uf[v];
            uf[v] = r;
            v = nx;
        }
        return r;
    };

    std::vector<std::vector<QEnt>> queue((size_t)V);
    std::vector<char> queue_ready((size_t)V, 0);
    std::vector<i64> lazy((size_t)V, 0);
    QCmp cmp;
    auto ensure_queue = [&](i32 c) {  // singleton components load their list on first use
        if (queue_ready[c]) return;
        queue_ready[c] = 1;
        if (c >= n) return;
        std::vector<QEnt>& q = queue[c];
        q.reserve((size_t)(g.off[c + 1] - g.off[c]));
        for (i64 k = g.off[c]; k < g.off[c + 1]; ++k) q.push_back({(i64)g.e[k].w, g.e[k].src, c});
        std::make_heap(q.begin(), q.end(), cmp);
    };

    // forest of choices
    std::vector<i32> f_src, f_dst, f_parent;
    f_src.reserve((size_t)2 * n);
    f_dst.reserve((size_t)2 * n);
    f_parent.reserve((size_t)2 * n);
    std::vector<i32> chosen((size_t)V, -1);        // forest node of the component's current choice
    std::vector<i32> pend_head((size_t)V, -1);     // cycle choices awaiting a parent, per component
    std::vector<i32> pend_next;                    // linked through forest-node ids
    pend_next.reserve((size_t)2 * n);
    std::vector<i32> leaf((size_t)n, -1);          // first choice made for each original vertex

    const i32 SETTLED = -1;
    std::vector<i32> mark((size_t)V, 0);  // 0 fresh, >0 id of the path it is on, SETTLED
    mark[n] = SETTLED;
    std::vector<i32> path;

    for (i32 s = 0; s < n; ++s) {
        i32 c = find(s);
        if (mark[c] != 0) continue;
        const i32 stamp = s + 1;
        path.clear();
        for (;;) {
            mark[c] = stamp;
            path.push_back(c);
            ensure_queue(c);
            std::vector<QEnt>& q = queue[c];
            QEnt best{};
            i32 from = -1;
            while (!q.empty()) {
                std::pop_heap(q.begin(), q.end(), cmp);
                best = q.back();
                q.pop_back();
                from = find(best.src);
                if (from != c) break;
                from = -1;  // edge fell inside the component
            }
            if (from < 0) {
                err = "arborescence: a component has no entering edge";
                return false;
            }
            lazy[c] -= best.key + lazy[c];  // reduce what remains by the cost just paid

            const i32 node = (i32)f_src.size();
            f_src.push_back(best.src);
            f_dst.push_back(best.dst);
            f_parent.push_back(-1);
            pend_next.push_back(-1);
            for (i32 ch = pend_head[c]; ch >= 0;) {
                const i32 nx = pend_next[ch];
                f_parent[ch] = node;
                pend_next[ch] = -1;
                ch = nx;
            }
            pend_head[c] = -1;
            chosen[c] = node;
            if (uf_size[c] == 1 && leaf[c] < 0) leaf[c] = node;

            if (mark[from] == SETTLED) {
                for (i32 pc : path) mark[pc] = SETTLED;
                break;
            }
            if (mark[from] == stamp) {
                // contract the tail of the path, from `from` to the end, into one component
                i32 base = from;  // member with the largest queue keeps it
                size_t k = path.size();
                do {
                    --k;
                    if (queue[path[k]].size() > queue[base].size()) base = path[k];
                } while (path[k] != from);
                const size_t first = k;
                i32 rep = path[first];
                i32 pend = -1;
                for (size_t j = first; j < path.size(); ++j) {
                    const i32 m = path[j];
                    // choices of the cycle members wait for the contracted component's choice
                    pend_next[chosen[m]] = pend;
                    pend = chosen[m];
                    if (m != base) {
                        std::vector<QEnt>& qb = queue[base];
                        const i64 shift = lazy[m] - lazy[base];
                        for (const QEnt& en : queue[m]) {
                            qb.push_back({en.key + shift, en.src, en.dst});
                            std::push_heap(qb.begin(), qb.end(), cmp);
                        }
                        std::vector<QEnt>().swap(queue[m]);
                    }
                    if (j > first) {  // union by size
                        i32 a = rep, b = m;
                        if (uf_size[a] < uf_size[b]) std::swap(a, b);
                        uf[b] = a;
                        uf_size[a] += uf_size[b];
                        rep = a;
                    }
                }
                if (rep != base) {
                    queue[rep].swap(queue[base]);
                    lazy[rep] = lazy[base];
                }
                queue_ready[rep] = 1;
                pend_head[rep] = pend;
                chosen[rep] = -1;
                mark[rep] = 0;
                path.resize(first);
                c = rep;
                continue;
            }
            c = from;  // fresh component: extend the path
        }
    }
    std::vector<std::vector<QEnt>>().swap(queue);

    // expansion
    const i32 F = (i32)f_src.size();
    std::vector<i32> child_off((size_t)F + 1, 0), child_idx;
    for (i32 x = 0; x < F; ++x)
        if (f_parent[x] >= 0) child_off[(size_t)f_parent[x] + 1]++;
    for (i32 x = 0; x < F; ++x) child_off[x + 1] += child_off[x];
    child_idx.resize((size_t)child_off[F]);
    {
        std::vector<i32> cur(child_off.begin(), child_off.end() - 1);
        for (i32 x = 0; x < F; ++x)
            if (f_parent[x] >= 0) child_idx[(size_t)cur[f_parent[x]]++] = x;
    }
    std::vector<char> gone((size_t)F, 0);
    std::vector<i32> roots;
    for (i32 x = F - 1; x >= 0; --x)
        if (f_parent[x] < 0) roots.push_back(x);
    out.parent.assign((size_t)n, -1);
    while (!roots.empty()) {
        const i32 top = roots.back();
        roots.pop_back();
        if (gone[top]) continue;
        const i32 v = f_dst[top];
        if (out.parent[v] >= 0) {
            err = "arborescence: vertex entered twice during expansion";
            return false;
        }
        out.parent[v] = f_src[top];
        i32 prev = -1;
        for (i32 x = leaf[v]; x >= 0; x = f_parent[x]) {
            gone[x] = 1;
            for (i32 k = child_off[x]; k < child_off[x + 1]; ++k) {
                const i32 ch = child_idx[k];
                if (ch != prev && !gone[ch]) {
                    f_parent[ch] = -1;
                    roots.push_back(ch);
                }
            }
            if (x == top) break;
            prev = x;
        }
    }
    for (i32 v = 0; v < n; ++v)
        if (out.parent[v] < 0) {
            err = "arborescence: vertex left without a parent";
            return false;
        }
    return true;
}

}  // namespace

// ------------------------------------------------------------------------------------------
// Built structure and the C ABI.
// ------------------------------------------------------------------------------------------
struct cbm_b200_built {
    i32 n = 0;
    std::vector<i32> parent;     // n
    std::vector<i32> mst_row;    // n+2
    std::vector<i32> mst_col;    // n
    std::vector<i32> bfs;        // n, visiting order
    std::vector<i32> d_crow;     // n+1
    std::vector<i32> d_col;
    std::vector<float> d_val;
    i64 n_candidates = 0;
    i32 n_root_children = 0;
    i32 depth = 0;
    double seconds[4] = {0, 0, 0, 0};
    int candidates_on_gpu = 0;
};

namespace {
int build_impl(const int32_t* row, const int32_t* col, int64_t nnz, int32_t n, int32_t alpha, const float* col_mul,
               int32_t n_threads, int device, cbm_b200_built** out);
}

extern "C" int cbm_b200_build(const int32_t* row, const int32_t* col, int64_t nnz, int32_t n,
                              int32_t alpha, const float* col_mul, int32_t n_threads,
                              cbm_b200_built** out) {
    return build_impl(row, col, nnz, n, alpha, col_mul, n_threads, -1, out);
}

extern "C" int cbm_b200_build_gpu(const int32_t* row, const int32_t* col, int64_t nnz, int32_t n,
                                  int32_t alpha, const float* col_mul, int32_t n_threads,
                                  int32_t device, cbm_b200_built** out) {
    if (device < 0) return cbm::fail(CBM_B200_ERR_ARG, "build_gpu: device must be a CUDA device ordinal");
    return build_impl(row, col, nnz, n, alpha, col_mul, n_threads, device, out);
}

namespace {
int build_impl(const int32_t* row, const int32_t* col, int64_t nnz, int32_t n, int32_t alpha, const float* col_mul,
               int32_t n_threads, int device, cbm_b200_built** out) {
    if (!out) return cbm::fail(CBM_B200_ERR_ARG, "build: out is NULL");
    *out = nullptr;
    if (n < 0 || nnz < 0 || (nnz > 0 && (!row || !col)))
        return cbm::fail(CBM_B200_ERR_ARG, "build: bad sizes or NULL index arrays");
    if (n >= INT32_MAX - 2) return cbm::fail(CBM_B200_ERR_ARG, "build: n too large for int32");
    for (i64 i = 0; i < nnz; ++i)
        if (row[i] < 0 || row[i] >= n || col[i] < 0 || col[i] >= n)
            return cbm::fail(CBM_B200_ERR_ARG, "build: index out of range at entry " +
                                                   std::to_string(i));
    const int prev_threads = omp_get_max_threads();
    if (n_threads > 0) omp_set_num_threads(n_threads);
    int status = CBM_B200_OK;
    try {
        // owned until it is handed to the caller: an exception on the way frees it
        std::unique_ptr<cbm_b200_built> b(new cbm_b200_built());
        b->n = n;
        const double t0 = now_s();
        Pattern a = make_csr(row, col, nnz, n);
        Arborescence arb;
        {
            Pattern at = transpose(a);
            bool on_gpu = false;
            Candidates g = make_candidates(a, at, alpha, device, &on_gpu);
            b->candidates_on_gpu = on_gpu ? 1 : 0;
            std::vector<i32>().swap(at.idx);
            b->n_candidates = g.total;
            const double t1 = now_s();
            b->seconds[0] = t1 - t0;
            std::string err;
            if (!solve_arborescence(g, n, arb, err)) {
                if (n_threads > 0) omp_set_num_threads(prev_threads);
                return cbm::fail(CBM_B200_ERR_FORMAT, err);
            }
            b->seconds[1] = now_s() - t1;
        }
        const double t2 = now_s();
        b->parent = arb.parent;

        // tree CSR over n+1 vertices; children in ascending id (cbm/cbm_extensions.cpp:274-286)
        b->mst_row.assign((size_t)n + 2, 0);
        for (i32 v = 0; v < n; ++v) b->mst_row[(size_t)arb.parent[v] + 1]++;
        for (i32 u = 0; u <= n; ++u) b->mst_row[u + 1] += b->mst_row[u];
        b->mst_col.resize((size_t)n);
        {
            std::vector<i32> cur(b->mst_row.begin(), b->mst_row.end() - 1);
            for (i32 v = 0; v < n; ++v) b->mst_col[(size_t)cur[arb.parent[v]]++] = v;
        }
        // breadth-first order from the virtual root (cbm/cbm_extensions.cpp:166-184)
        b->bfs.reserve((size_t)n);
        std::vector<i32> level((size_t)n + 1, 0);
        {
            size_t head = 0;
            std::vector<i32> order;
            order.reserve((size_t)n + 1);
            order.push_back(n);
            while (head < order.size()) {
                const i32 u = order[head++];
                for (i32 k = b->mst_row[u]; k < b->mst_row[u + 1]; ++k) {
                    const i32 v = b->mst_col[k];
                    level[v] = level[u] + 1;
                    b->depth = std::max(b->depth, level[v]);
                    order.push_back(v);
                }
            }
            if ((i32)order.size() != n + 1) {
                if (n_threads > 0) omp_set_num_threads(prev_threads);
                return cbm::fail(CBM_B200_ERR_FORMAT, "build: tree does not span every row");
            }
            b->bfs.assign(order.begin() + 1, order.end());
        }
        b->n_root_children = b->mst_row[n + 1] - b->mst_row[n];

        // deltas by sorted merge (cbm/cbm_extensions.cpp:186-261; values :504-584 when col_mul)
        b->d_crow.assign((size_t)n + 1, 0);
        std::vector<i32> dlen((size_t)n, 0);
#pragma omp parallel for schedule(dynamic, 512)
        for (i32 v = 0; v < n; ++v) {
            const i32 u = arb.parent[v];
            if (u == n) {
                dlen[v] = a.len(v);
                continue;
            }
            const i32 *pu = a.idx.data() + a.ptr[u], *eu = a.idx.data() + a.ptr[u + 1];
            const i32 *pv = a.idx.data() + a.ptr[v], *ev = a.idx.data() + a.ptr[v + 1];
            i32 cntd = 0;
            while (pu < eu && pv < ev) {
                if (*pu == *pv) {
                    ++pu;
                    ++pv;
                } else if (*pu > *pv) {
                    ++cntd;
                    ++pv;
                } else {
                    ++cntd;
                    ++pu;
                }
            }
            dlen[v] = cntd + (i32)(eu - pu) + (i32)(ev - pv);
        }
        i64 total = 0;
        for (i32 v = 0; v < n; ++v) {
            total += dlen[v];
            if (total > INT32_MAX) {
                if (n_threads > 0) omp_set_num_threads(prev_threads);
                return cbm::fail(CBM_B200_ERR_ARG, "build: more than 2^31-1 delta entries");
            }
            b->d_crow[v + 1] = (i32)total;
        }
        b->d_col.resize((size_t)total);
        b->d_val.resize((size_t)total);
#pragma omp parallel for schedule(dynamic, 512)
        for (i32 v = 0; v < n; ++v) {
            const i32 u = arb.parent[v];
            i32* oc = b->d_col.data() + b->d_crow[v];
            float* ov = b->d_val.data() + b->d_crow[v];
            const i32 *pv = a.idx.data() + a.ptr[v], *ev = a.idx.data() + a.ptr[v + 1];
            auto emit = [&](i32 c, bool plus) {
                const float m = col_mul ? col_mul[c] : 1.0f;
                *oc++ = c;
                *ov++ = plus ? m : -m;
            };
            if (u == n) {
                for (; pv < ev; ++pv) emit(*pv, true);
                continue;
            }
            const i32 *pu = a.idx.data() + a.ptr[u], *eu = a.idx.data() + a.ptr[u + 1];
            while (pu < eu && pv < ev) {
                if (*pu == *pv) {
                    ++pu;
                    ++pv;
                } else if (*pu > *pv) {
                    emit(*pv++, true);
                } else {
                    emit(*pu++, false);
                }
            }
            // the two tails are disjoint in column range, so emitting the lower one first keeps
            // the row's columns ascending
            for (; pu < eu; ++pu) emit(*pu, false);
            for (; pv < ev; ++pv) emit(*pv, true);
        }
        b->seconds[2] = now_s() - t2;
        b->seconds[3] = now_s() - t0;
        *out = b.release();
    } catch (const std::bad_alloc&) {
        status = cbm::fail(CBM_B200_ERR_ALLOC, "build: out of host memory");
    }
    if (n_threads > 0) omp_set_num_threads(prev_threads);
    return status;
}
}  // namespace

extern "C" int cbm_b200_built_candidates_on_gpu(const cbm_b200_built* b) { return b ? b->candidates_on_gpu : 0; }

extern "C" int cbm_b200_built_info(const cbm_b200_built* b, int64_t* n_delta,
                                   int64_t* n_candidates, int32_t* n_root_children,
                                   int32_t* depth, double* seconds) {
    if (!b) return cbm::fail(CBM_B200_ERR_ARG, "built_info: NULL handle");
    if (n_delta) *n_delta = (i64)b->d_col.size();
    if (n_candidates) *n_candidates = b->n_candidates;
    if (n_root_children) *n_root_children = b->n_root_children;
    if (depth) *depth = b->depth;
    if (seconds) std::memcpy(seconds, b->seconds, sizeof(b->seconds));
    return CBM_B200_OK;
}

extern "C" int cbm_b200_built_export_csr(const cbm_b200_built* b, int32_t* mst_row,
                                         int32_t* mst_col, int32_t* delta_crow,
                                         int32_t* delta_col, float* delta_val, int32_t* parent) {
    if (!b) return cbm::fail(CBM_B200_ERR_ARG, "built_export_csr: NULL handle");
    if (!mst_row || !delta_crow || (b->n > 0 && !mst_col) ||
        (!b->d_col.empty() && (!delta_col || !delta_val)))
        return cbm::fail(CBM_B200_ERR_ARG, "built_export_csr: NULL output array");
    std::copy(b->mst_row.begin(), b->mst_row.end(), mst_row);
    std::copy(b->mst_col.begin(), b->mst_col.end(), mst_col);
    std::copy(b->d_crow.begin(), b->d_crow.end(), delta_crow);
    std::copy(b->d_col.begin(), b->d_col.end(), delta_col);
    std::copy(b->d_val.begin(), b->d_val.end(), delta_val);
    if (parent) std::copy(b->parent.begin(), b->parent.end(), parent);
    return CBM_B200_OK;
}

extern "C" int cbm_b200_built_export_coo(const cbm_b200_built* b, int32_t* delta_row,
                                         int32_t* delta_col, float* delta_val) {
    if (!b) return cbm::fail(CBM_B200_ERR_ARG, "built_export_coo: NULL handle");
    if (!b->d_col.empty() && (!delta_row || !delta_col || !delta_val))
        return cbm::fail(CBM_B200_ERR_ARG, "built_export_coo: NULL output array");
    size_t o = 0;
    for (i32 v : b->bfs)
        for (i32 k = b->d_crow[v]; k < b->d_crow[v + 1]; ++k, ++o) {
            delta_row[o] = v;
            delta_col[o] = b->d_col[k];
            delta_val[o] = b->d_val[k];
        }
    return CBM_B200_OK;
}

extern "C" void cbm_b200_built_free(cbm_b200_built* b) { delete b; }
