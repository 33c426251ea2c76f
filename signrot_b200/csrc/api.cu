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

int tc_device_status(int *out, bool clear);
int grouped_device_status(int *out, bool clear);
int tc2_device_status(int *out, bool clear);
int tc3_device_status(int *out, bool clear);

}  // namespace sr

extern "C" {

const char *sr_last_error(void) { return sr::last_error_buffer(); }

int sr_version(void) { return SR_VERSION; }

int sr_device_status(int *status, int clear) {
    SR_REQUIRE(status != nullptr, SR_ERR_INVALID, "device_status: null pointer");
    int a = 0, b = 0;
    int rc = sr::tc_device_status(&a, clear != 0);
    if (rc) return rc;
    rc = sr::grouped_device_status(&b, clear != 0);
    if (rc) return rc;
    int c = 0;
    rc = sr::tc2_device_status(&c, clear != 0);
    if (rc) return rc;
    int d = 0;
    rc = sr::tc3_device_status(&d, clear != 0);
    if (rc) return rc;
    *status = a ? a : (b ? b : (c ? c : d));
    return SR_OK;
}

}  // extern "C"
