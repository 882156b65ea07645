// Backend-parameterised operator tests: this file only names the tests the B200 backend does not
// run (docs/Backends.md, "Backend Parameterized Tests").  Everything on the quantized inference
// path is enabled -- including the 4-bit and fp16 fused-rowwise tests the CPU backend blacklists
// (lib/Backends/CPU/tests/CPUOperatorTest.cpp:254-292).
#include "tests/unittests/BackendTestUtils.h"

using namespace glow;

std::set<std::string> glow::backendTestBlacklist = {
    // float and training operators are outside this backend (isOpSupported refuses them)
    "Conv3DQuantizedTest/0", "less_float16Cases/0", "less_int64Cases/0", "ResizeNearest_Float/0", "ResizeBilinear_Float/0",
    "LSTMUnitFP16/0", "PyTorchLSTMFP16/0", "GRU/0", "BatchedGather/0", "CumSum1D/0", "ArgMaxKeepDim/0",
};
