// Last-error text of the library (host side only).
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

void sb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

extern "C" const char* sb_last_error() { return g_error; }

namespace sb {
bool pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("SOCRATES_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}
}  // namespace sb

extern "C" int sb_abi_version() { return 1; }
