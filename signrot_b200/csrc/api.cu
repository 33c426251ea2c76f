// Error reporting and library identification for the C ABI.
#include "common.cuh"
#include <cstring>

namespace sr {

char *last_error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

int grouped_device_status(int *out, bool clear);
int tc3_device_status(int *out, bool clear);
int peer_device_status(int *out, bool clear);
int rotate_umma_device_status(int *out, bool clear);
int rotate_had28_umma_device_status(int *out, bool clear);
int launch_bounded_wait_probe(long long budget_cycles, cudaStream_t st);

}  // namespace sr

extern "C" {

const char *sr_last_error(void) { return sr::last_error_buffer(); }

int sr_version(void) { return SR_VERSION; }

int sr_device_status(int *status, int clear) {
    SR_REQUIRE(status != nullptr, SR_ERR_INVALID, "device_status: null pointer");
    int a = 0, b = 0;
    int rc = sr::tc3_device_status(&a, clear != 0);
    if (rc) return rc;
    rc = sr::grouped_device_status(&b, clear != 0);
    if (rc) return rc;
    int c = 0;
    rc = sr::peer_device_status(&c, clear != 0);
    if (rc) return rc;
    int d = 0;
    rc = sr::rotate_umma_device_status(&d, clear != 0);
    if (rc) return rc;
    int e = 0;
    rc = sr::rotate_had28_umma_device_status(&e, clear != 0);
    if (rc) return rc;
    *status = a ? a : (b ? b : (c ? c : (d ? d : e)));
    return SR_OK;
}

int sr_selftest_bounded_wait(int64_t budget_cycles, void *stream) {
    SR_REQUIRE(budget_cycles >= 1000 && budget_cycles <= 10000000, SR_ERR_INVALID,
               "selftest_bounded_wait: budget of %lld cycles outside 1e3 .. 1e7", (long long)budget_cycles);
    return sr::launch_bounded_wait_probe((long long)budget_cycles, sr::as_stream(stream));
}

}  // extern "C"
