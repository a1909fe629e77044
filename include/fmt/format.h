// fmt/format.h of the stand-in: everything lives in core.h.
#pragma once
#include "core.h"
