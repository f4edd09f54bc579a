// TEST INFRASTRUCTURE — stand-in for <arbok/tarjan/tarjan_pq.h> of the arbok library, which the
// reference vendors as a git submodule that is not present offline.  It offers the four members
// cbm/cbm_extensions.cpp uses (constructor, create_edge, run, reconstruct; call sites at
// cbm/cbm_extensions.cpp:109-148 and :427-468) over an own implementation of the published
// minimum-cost arborescence algorithm (Chu-Liu/Edmonds in Tarjan's formulation: grow a path of
// cheapest incoming edges, contract cycles with mergeable heaps carrying lazy key offsets, then
// expand the contraction forest from the root).  Any minimum-cost arborescence has the same total
// weight; which of several optimal trees comes out (tie-breaking) is implementation-defined here as
// it is in arbok.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <utility>
#include <vector>

namespace arbok {

class TarjanPQ {
public:
    TarjanPQ(int n_vertices, int n_edges_hint) : n_(n_vertices) {
        from_.reserve((size_t)n_edges_hint);
        to_.reserve((size_t)n_edges_hint);
        w_.reserve((size_t)n_edges_hint);
    }

    // Edges are numbered in creation order; reconstruct() answers with these numbers.
    void create_edge(int from, int to, int weight) {
        from_.push_back(from);
        to_.push_back(to);
        w_.push_back(weight);
    }

    // Contraction phase.  Returns the weight of a minimum-cost arborescence rooted at `root`.
    long long run(int root) {
        const int m = (int)from_.size();
        const int max_nodes = 2 * n_;
        key_.assign((size_t)m, 0);
        lazy_.assign((size_t)m, 0);
        lc_.assign((size_t)m, -1);
        rc_.assign((size_t)m, -1);
        rank_.assign((size_t)m, 1);
        heap_.assign((size_t)max_nodes, -1);
        dsu_.resize((size_t)max_nodes);
        for (int i = 0; i < max_nodes; ++i) dsu_[i] = i;
        up_.assign((size_t)max_nodes, -1);
        kids_.assign((size_t)max_nodes, {});
        enter_.assign((size_t)max_nodes, -1);
        n_nodes_ = n_;
        for (int e = 0; e < m; ++e) {
            if (to_[e] == root || from_[e] == to_[e]) continue;
            key_[e] = w_[e];
            heap_[to_[e]] = meld(heap_[to_[e]], e);
        }
        std::vector<char> state((size_t)max_nodes, 0);  // 0 untouched, 1 on the path, 2 settled
        state[root] = 2;
        long long total = 0;
        std::vector<int> path;
        for (int start = 0; start < n_; ++start) {
            int a = find(start);
            if (state[a] != 0) continue;
            path.clear();
            while (state[a] == 0) {
                state[a] = 1;
                path.push_back(a);
                int e = -1;
                for (;;) {  // cheapest edge that really enters the (super)vertex a
                    e = heap_[a];
                    if (e < 0) throw std::runtime_error("TarjanPQ: a vertex cannot be reached from the root");
                    settle(e);
                    heap_[a] = meld(lc_[e], rc_[e]);
                    lc_[e] = rc_[e] = -1;
                    if (find(from_[e]) != a) break;
                }
                enter_[a] = e;
                total += key_[e];
                if (heap_[a] >= 0) lazy_[heap_[a]] -= key_[e];
                int b = find(from_[e]);
                if (state[b] == 1) {  // the path closed a cycle b ... a: contract it
                    const int c = n_nodes_++;
                    int h = -1;
                    for (;;) {
                        const int v = path.back();
                        path.pop_back();
                        dsu_[v] = c;
                        up_[v] = c;
                        kids_[c].push_back(v);
                        h = meld(h, heap_[v]);
                        heap_[v] = -1;
                        if (v == b) break;
                    }
                    heap_[c] = h;
                    b = c;  // state 0: it joins the path on the next turn
                }
                a = b;
            }
            for (int v : path) state[v] = 2;
        }
        root_ = root;
        return total;
    }

    // Expansion phase: the edge numbers of the arborescence found by run(), one per non-root vertex.
    std::vector<int> reconstruct(int root) {
        if (root != root_) throw std::runtime_error("TarjanPQ: reconstruct() root differs from run()");
        std::vector<int> chosen((size_t)n_, -1);
        std::vector<int> todo;
        for (int v = 0; v < n_nodes_; ++v)
            if (up_[v] < 0 && v != root) todo.push_back(v);
        while (!todo.empty()) {
            const int top = todo.back();
            todo.pop_back();
            const int e = enter_[top];
            int x = to_[e];
            chosen[x] = e;
            while (x != top) {  // open every contracted cycle on the way up: its other members keep their cycle edge
                const int p = up_[x];
                for (int c : kids_[p])
                    if (c != x) {
                        up_[c] = -1;
                        todo.push_back(c);
                    }
                x = p;
            }
        }
        std::vector<int> out;
        out.reserve((size_t)n_ - 1);
        for (int v = 0; v < n_; ++v)
            if (v != root) out.push_back(chosen[v]);
        return out;
    }

private:
    int find(int v) {
        int r = v;
        while (dsu_[r] != r) r = dsu_[r];
        while (dsu_[v] != r) {
            const int nx = dsu_[v];
            dsu_[v] = r;
            v = nx;
        }
        return r;
    }
    void settle(int e) {  // apply the pending offset of e and hand it to its children
        if (lazy_[e] != 0) {
            key_[e] += lazy_[e];
            if (lc_[e] >= 0) lazy_[lc_[e]] += lazy_[e];
            if (rc_[e] >= 0) lazy_[rc_[e]] += lazy_[e];
            lazy_[e] = 0;
        }
    }
    // leftist heap: the recursion follows right spines only, which are logarithmic
    int meld(int a, int b) {
        if (a < 0) return b;
        if (b < 0) return a;
        settle(a);
        settle(b);
        if (key_[b] < key_[a]) std::swap(a, b);
        rc_[a] = meld(rc_[a], b);
        const int rl = lc_[a] >= 0 ? rank_[lc_[a]] : 0, rr = rc_[a] >= 0 ? rank_[rc_[a]] : 0;
        if (rl < rr) std::swap(lc_[a], rc_[a]);
        rank_[a] = (rl < rr ? rl : rr) + 1;
        return a;
    }

    int n_, n_nodes_ = 0, root_ = -1;
    std::vector<int> from_, to_, w_;
    std::vector<long long> key_, lazy_;
    std::vector<int> lc_, rc_, rank_, heap_, dsu_, up_, enter_;
    std::vector<std::vector<int>> kids_;
};

}  // namespace arbok
