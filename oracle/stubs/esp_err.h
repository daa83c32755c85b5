#pragma once
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
typedef int esp_err_t;
#define ESP_OK 0
#define ESP_FAIL -1
#define ESP_ERR_NO_MEM 0x101
#define ESP_ERR_INVALID_ARG 0x102
#define ESP_ERR_INVALID_STATE 0x103
#define ESP_ERR_NOT_FOUND 0x105
#define ESP_ERR_NOT_SUPPORTED 0x106
#define ESP_ERROR_CHECK(x) do { if ((x) != ESP_OK) abort(); } while (0)
#define ESP_RETURN_ON_ERROR(x, tag, fmt, ...) do { esp_err_t e_ = (x); if (e_ != ESP_OK) return e_; } while (0)
#define ESP_RETURN_ON_FALSE(c, err, tag, fmt, ...) do { if (!(c)) return (err); } while (0)
