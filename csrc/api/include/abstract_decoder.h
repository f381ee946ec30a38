// The reference's header name (include/abstract_decoder.h); the declarations live in csrc/api/xft/abstract_decoder.h.
#pragma once
#include "../xft/abstract_decoder.h"
