#pragma once
#include "esp_err.h"
typedef uint32_t esp_paddr_t;
typedef enum { MMU_TARGET_FLASH0 = 1, MMU_TARGET_PSRAM0 = 2 } mmu_target_t;
