// The reference's header name (include/abstract_searcher.h); the declarations live in csrc/api/xft/abstract_searcher.h.
#pragma once
#include "../xft/abstract_searcher.h"
