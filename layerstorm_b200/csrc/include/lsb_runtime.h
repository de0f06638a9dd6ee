// C ABI shared by the host runtime library (liblsb200_runtime.so) and its Python bindings.
#pragma once
#include <stdint.h>

#define LSB_RT_API __attribute__((visibility("default")))

// Error codes returned by runtime entry points (0 = ok).
enum {
    LSB_OK = 0,
    LSB_ERR_ARG = -1,
    LSB_ERR_NOT_FOUND = -2,
    LSB_ERR_EXISTS = -3,
    LSB_ERR_POOL_EXHAUSTED = -4,   // no free KV pages (the reference's kKvPoolExhausted)
    LSB_ERR_FROZEN = -5,
    LSB_ERR_SHARED = -6,
    LSB_ERR_FULL = -7,
    LSB_ERR_BUSY = -8,
    LSB_ERR_IO = -9,
    LSB_ERR_FORMAT = -10,
};
