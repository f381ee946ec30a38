// The reference's header name (include/dtype.h); the declarations live in csrc/api/xft/dtype.h.
#pragma once
#include "../xft/dtype.h"
