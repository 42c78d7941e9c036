// Error plumbing shared by the C ABI translation units.
#pragma once
#include "common.cuh"
#include <string>
#include <exception>

namespace mk {

std::string& last_error_slot();   // thread-local message behind mk_last_error()
void require_device();            // throws when no CUDA device is usable (there is no CPU fallback)

struct KvExhausted : std::runtime_error {
    using std::runtime_error::runtime_error;
};

template <typename F>
int32_t guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const KvExhausted& e) {
        last_error_slot() = e.what();
        return 1;
    } catch (const std::exception& e) {
        last_error_slot() = e.what();
        return -1;
    } catch (...) {
        last_error_slot() = "unknown error";
        return -1;
    }
}

}  // namespace mk
