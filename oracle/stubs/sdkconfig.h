/* Host stand-in for ESP-IDF's generated sdkconfig.h (oracle build only).
 * No CONFIG_IDF_TARGET_* is defined, so every *_BOOST switch of the reference
 * is 0 and only its generic C kernels (round-half-up) are compiled. */
#pragma once
#include <assert.h>
#include <limits.h>
#include <stdint.h>
#include <stddef.h>
#define CONFIG_FREERTOS_NUMBER_OF_CORES 1
#define CONFIG_LOG_MAXIMUM_LEVEL 1
