// Enumerations and small helpers shared by the host layer.  Names and numeric values follow
// ESP-DL (esp-dl/dl/dl_define.hpp:47-143) so that code written against its headers reads the same.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstdlib>

typedef int esp_err_t;
#ifndef ESP_OK
#define ESP_OK 0
#define ESP_FAIL -1
#endif

namespace dl {
void log_message(char level, const char *tag, const char *fmt, ...);
}
#define ESP_LOGE(tag, ...) ::dl::log_message('E', tag, __VA_ARGS__)
#define ESP_LOGW(tag, ...) ::dl::log_message('W', tag, __VA_ARGS__)
#define ESP_LOGI(tag, ...) ::dl::log_message('I', tag, __VA_ARGS__)

#define DL_SCALE(exponent) (((exponent) > 0) ? (float)(1 << (exponent)) : ((float)1.0 / (float)(1 << -(exponent))))
#define DL_RESCALE(exponent) (((exponent) > 0) ? ((float)1.0 / (float)(1 << (exponent))) : (float)(1 << -(exponent)))

namespace dl {
typedef enum {
    QUANT_TYPE_NONE,
    QUANT_TYPE_FLOAT32,
    QUANT_TYPE_SYMM_8BIT,
    QUANT_TYPE_SYMM_16BIT,
    QUANT_TYPE_SYMM_32BIT,
} quant_type_t;

typedef enum { Linear, ReLU, LeakyReLU, PReLU } activation_type_t;
typedef enum { RESIZE_NEAREST, RESIZE_LINEAR, RESIZE_CUBIC } resize_mode_t;

typedef enum {
    RUNTIME_MODE_AUTO = 0,
    RUNTIME_MODE_SINGLE_CORE = 1,
    RUNTIME_MODE_MULTI_CORE = 2,
} runtime_mode_t;

// Rounding of requantisation shifts: the reference fixes it at build time per chip
// (esp-dl/dl/dl_define_private.hpp:44-48); here it is a property of the loaded model.
typedef enum { ROUND_HALF_UP = 0, ROUND_HALF_EVEN = 1 } round_mode_t;

// Memory "capabilities" of the reference's allocator; kept so that signatures match. All device
// tensors live in HBM.
#define MALLOC_CAP_DEFAULT (1 << 12)
#define MALLOC_CAP_INTERNAL (1 << 11)
#define MALLOC_CAP_SPIRAM (1 << 10)
} // namespace dl
