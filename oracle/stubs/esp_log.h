#pragma once
#include "esp_err.h"
#include <stdio.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef enum { ESP_LOG_NONE, ESP_LOG_ERROR, ESP_LOG_WARN, ESP_LOG_INFO, ESP_LOG_DEBUG, ESP_LOG_VERBOSE } esp_log_level_t;
#define ESP_LOGE(tag, fmt, ...) fprintf(stderr, "E (%s) " fmt "\n", tag, ##__VA_ARGS__)
#define ESP_LOGW(tag, fmt, ...) do { if (getenv("ESPDL_REF_VERBOSE")) fprintf(stderr, "W (%s) " fmt "\n", tag, ##__VA_ARGS__); } while (0)
#define ESP_LOGI(tag, fmt, ...) do { if (getenv("ESPDL_REF_VERBOSE")) fprintf(stderr, "I (%s) " fmt "\n", tag, ##__VA_ARGS__); } while (0)
#define ESP_LOGD(tag, fmt, ...) do { } while (0)
#define ESP_LOGV(tag, fmt, ...) do { } while (0)
static inline void esp_log_level_set(const char *tag, esp_log_level_t l) { (void)tag; (void)l; }
#ifdef __cplusplus
}
#endif
