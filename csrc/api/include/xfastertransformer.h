// Umbrella header under the reference's name (include/xfastertransformer.h): a program written against the reference
// compiles with -I csrc/api/include and links libxft_b200_core.so.
#pragma once
#include "abstract_decoder.h"
#include "abstract_searcher.h"
#include "dtype.h"
#include "layers_attention.h"
#include "layers_decoder.h"
#include "layers_gemm.h"
#include "layers_mlp.h"
#include "layers_norm.h"
#include "layers_rotary_embedding.h"
#include "layers_token_embedding.h"
#include "models.h"
