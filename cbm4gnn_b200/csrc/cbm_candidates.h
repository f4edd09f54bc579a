// Interface between the host builder (cbm_builder.cpp) and its GPU candidate search
// (cbm_candidates.cu).
#ifndef CBM_CANDIDATES_H
#define CBM_CANDIDATES_H

#include <cstdint>
#include <string>
#include <vector>

namespace cbm {

struct CandTriple {
    int32_t src, dst, w;  // candidate edge src -> dst with weight h(src, dst)
};

// Candidate edges between real rows (the virtual root's edges are added by the caller).
// row_ptr / row_rank: the pattern's rows with every column replaced by its rank in the
// rare-to-frequent order and sorted ascending; col_of_rank: rank -> column; col_ptr / col_rows: the
// column lists.  Parents whose prefix is too long for the GPU's 16-bit counters come back in
// left_to_host.  Returns 0 on success; on failure `err` says why and the caller falls back.
int gpu_candidates(int device, int32_t n, int32_t alpha, const int64_t* row_ptr, const int32_t* row_rank,
                   const int32_t* col_of_rank, const int64_t* col_ptr, const int32_t* col_rows,
                   std::vector<CandTriple>& out, std::vector<int32_t>& left_to_host, std::string& err);

}  // namespace cbm

#endif
