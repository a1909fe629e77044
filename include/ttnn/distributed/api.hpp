// Forwards to the B200 stand-in for the TTNN / tt-metalium API (see ttnn_b200/ttnn_b200.hpp).
#pragma once
#include "../../ttnn_b200/ttnn_b200.hpp"
