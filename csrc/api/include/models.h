// The reference's header name (include/models.h); the declarations live in csrc/api/xft/models.h.
#pragma once
#include "../xft/models.h"
