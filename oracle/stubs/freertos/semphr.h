#pragma once
#include "freertos/FreeRTOS.h"
