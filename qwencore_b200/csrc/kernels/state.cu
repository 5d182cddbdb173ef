// Process-wide shape selection and the sticky device status word.
#include "common.cuh"

#include "../../../include/qwc_abi.h"

namespace qwc {

namespace {

// Defaults reproduce the reference constants (cuda/delta_net.cu:36, cuda/paged_attention.cu:21).
Shape g_shape = {48, 64};

// [0] the sticky status word; [2], [3] what the first failed wait for a peer looked for and found (tags)
__device__ int g_status_word[4] = {0, 0, 0, 0};


int* g_status_ptrs[kMaxDevices] = {};

}  // namespace

Shape current_shape() { return g_shape; }

int* status_ptr() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        return nullptr;
    }
    if (g_status_ptrs[device] == nullptr) {
        void* address = nullptr;
        if (cudaGetSymbolAddress(&address, g_status_word) != cudaSuccess) {
            return nullptr;
        }
        g_status_ptrs[device] = static_cast<int*>(address);
    }
    return g_status_ptrs[device];
}

}  // namespace qwc

extern "C" int qwc_configure(const qwc_shape* shape) {
    if (shape == nullptr || (shape->delta_value_heads != 32 && shape->delta_value_heads != 48) ||
        (shape->kv_page_size != 16 && shape->kv_page_size != 64)) {
        return cudaErrorInvalidValue;
    }
    qwc::g_shape.delta_value_heads = shape->delta_value_heads;
    qwc::g_shape.kv_page_size = shape->kv_page_size;
    return cudaSuccess;
}

extern "C" void qwc_get_shape(qwc_shape* shape) {
    if (shape != nullptr) {
        shape->delta_value_heads = qwc::g_shape.delta_value_heads;
        shape->kv_page_size = qwc::g_shape.kv_page_size;
    }
}

extern "C" int qwc_device_status(void) {
    int* word = qwc::status_ptr();
    if (word == nullptr) {
        return -1;
    }
    int value = 0;
    if (cudaMemcpy(&value, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        return -1;
    }
    return value;
}

extern "C" int qwc_device_status_reset(void) {
    int* word = qwc::status_ptr();
    if (word == nullptr) {
        return cudaErrorInvalidValue;
    }
    return cudaMemset(word, 0, 4 * sizeof(int));
}

extern "C" int qwc_device_status_detail(uint32_t* expected_and_found) {
    int* word = qwc::status_ptr();
    if (word == nullptr || expected_and_found == nullptr) {
        return cudaErrorInvalidValue;
    }
    return cudaMemcpy(expected_and_found, word + 2, 2 * sizeof(int), cudaMemcpyDeviceToHost);
}

extern "C" int qwc_device_status_set(int code) {
    int* word = qwc::status_ptr();
    if (word == nullptr) {
        return cudaErrorInvalidValue;
    }
    return cudaMemcpy(word, &code, sizeof(int), cudaMemcpyHostToDevice);
}

extern "C" int qwc_device_status_copy(void* destination, qwc_stream stream) {
    int* word = qwc::status_ptr();
    if (word == nullptr || destination == nullptr) {
        return cudaErrorInvalidValue;
    }
    return cudaMemcpyAsync(destination, word, sizeof(int), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
}
