// Version / size handshakes and the thread-local error text of the C ABI
// (upstream convention: native/roce_bridge.cpp:22-104, native/xgrammar/bridge.h:9-14).
#include "common.cuh"

namespace gf {
std::string &last_error() {
    thread_local std::string e;
    return e;
}
int fail(const std::string &msg) {
    last_error() = msg;
    return -1;
}
int fail_cuda(cudaError_t e, const char *what) {
    // upstream formats driver errors as "CUDA {code} {name}: {msg}" (src/cuda.rs:102-123)
    last_error() = "CUDA " + std::to_string((int)e) + " " + cudaGetErrorName(e) + ": " + cudaGetErrorString(e) + " (" + what + ")";
    return -1;
}
}  // namespace gf

extern "C" int glmflash_abi_version(void) { return GLMFLASH_ABI_VERSION; }
extern "C" size_t glmflash_config_bytes(void) { return sizeof(glmflash_config); }
extern "C" size_t glmflash_weights_bytes(void) { return sizeof(glmflash_weights); }
extern "C" const char *glmflash_error(void) { return gf::last_error().c_str(); }
