#pragma once
#include "esp_err.h"
#include "esp_heap_caps.h"
