#pragma once
#include "esp_err.h"
