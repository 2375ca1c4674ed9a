// C++ host API of flexllm_b200: thin inline wrappers over the C ABI (include/flexllm_b200.h) that keep
// the names of FlexLLM's operator templates (Modules/*.h). Where the reference passes TAPA streams
// and compile-time lane counts, these take device pointers, run-time sizes and a CUDA stream; the
// return value is the C ABI's status code (the reference's operators return void and cannot fail).
#pragma once
#include <cstddef>
#include <cstdint>

#include "../flexllm_b200.h"

namespace flexllm {
using stream_t = void*;  // cudaStream_t
inline const char* status_string(int st) { return flexllm_status_string(st); }
}  // namespace flexllm
