// Acceptance check of the source-level drop-in: compiles the REFERENCE project's own, unmodified
// nn_operators/layernorm/main.cu (taken from the reference checkout at build time, -DKO_REFERENCE_MAIN=...)
// against THIS repository's headers.  The reference driver includes its headers by relative path, so
// this wrapper includes ours first and pre-defines the reference headers' include guards: when the
// driver then includes its own copies they are empty and every name resolves to our implementation.
// Test infrastructure only (built by `make -C oracle compat` into oracle/_ref/).
#include <cstdint>
#include <iostream>
#include <string>

#include "../../kernel_optimization_b200/common/common.h"
#include "../../kernel_optimization_b200/common/functors.h"
#include "../../kernel_optimization_b200/common/tensor.h"
#include "../../kernel_optimization_b200/nn_operators/layernorm/layernorm.h"

#define KERNEL_OPTIMIZATION_COMMON_H
#define KERNEL_OPTIMIZATION_FUNCTORS_H
#define KERNEL_OPTIMIZATION_TENSOR_H
#define KERNEL_OPTIMIZATION_LAYERNORM_H

#include KO_REFERENCE_MAIN
