// Back end: the reference prints CUDA C source for every "gpu" function
// (src/Backend/CUDA.cc:1170-1182).  The kernels here are pre-built, so the generated text is
// the dispatch plan: one line per kernel launch naming the C-ABI entry point and its
// arguments, in execution order.
#pragma once

#include <string>

namespace KernelCodeGen {

struct Module;
std::string CUDAGen(Module& module);

}  // namespace KernelCodeGen
