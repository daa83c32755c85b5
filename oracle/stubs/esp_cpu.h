#pragma once
#include <stdint.h>
#include "esp_timer.h"
typedef uint32_t esp_cpu_cycle_count_t;
static inline esp_cpu_cycle_count_t esp_cpu_get_cycle_count(void) { return (esp_cpu_cycle_count_t)(esp_timer_get_time() * 240); }
