// Enums of the operator API live in Frontend/Types.h.
#pragma once
#include "Frontend/Types.h"
