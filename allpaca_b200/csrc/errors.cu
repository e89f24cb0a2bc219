// Per-thread text of the last failed call of this library.
#include "common.cuh"
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

static thread_local char g_error[512] = "";

void ap_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

AP_EXPORT const char* ap_last_error(void) { return g_error; }

bool ap_pdl_enabled() {
    static int state = -1;
    if (state < 0) {
        const char* v = getenv("ALLPACA_PDL");
        state = (v && v[0] == '0') ? 0 : 1;
    }
    return state == 1;
}

// Compile-time facts the Python side checks after loading.
AP_EXPORT int ap_abi_version(void) { return 1; }
