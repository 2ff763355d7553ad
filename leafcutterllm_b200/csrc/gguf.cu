// GGUF v3 file loading (Engine::load(path), rust/src/inference/engine.rs:18-49).
#include "lc_kernels.h"

using namespace lc;

extern "C" int32_t lc_model_load_gguf(const char* path, const lc_model_config* overrides, lc_model** out) {
    (void)path; (void)overrides; (void)out;
    set_error("lc_model_load_gguf is not implemented yet; create the model and hand over tensors with lc_model_set_tensor");
    return LC_ERR_UNSUPPORTED;
}
