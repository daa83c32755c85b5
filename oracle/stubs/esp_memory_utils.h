#pragma once
#include "esp_heap_caps.h"
static inline bool esp_ptr_external_ram(const void *p) { (void)p; return false; }
static inline bool esp_ptr_in_drom(const void *p) { (void)p; return false; }
static inline bool esp_ptr_internal(const void *p) { (void)p; return true; }
static inline bool esp_ptr_in_tcm(const void *p) { (void)p; return false; }
