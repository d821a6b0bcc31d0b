// The Log switch lives in Frontend/Types.h.
#pragma once
#include "Frontend/Types.h"
