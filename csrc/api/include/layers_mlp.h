// The reference's header name (include/layers_mlp.h); the layer-level calls are declared together in csrc/api/xft/layers.h
// (device pointers here, host pointers there).
#pragma once
#include "../xft/layers.h"
