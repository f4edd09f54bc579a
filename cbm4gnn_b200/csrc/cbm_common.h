// Error plumbing shared by the host builder and the CUDA engine.
// The reference reports native failures by printing and calling exit(-1)
// (cbm/helpers.hpp:57-85); here every failure becomes a status code plus a per-thread message.
#ifndef CBM_COMMON_H
#define CBM_COMMON_H

#include <string>

namespace cbm {

std::string& last_error_slot();

inline int fail(int code, const std::string& msg) {
    last_error_slot() = msg;
    return code;
}

}  // namespace cbm

#endif
