// Shared by the TenniS operator classes of the B200 int8 path.
#ifndef TENNIS_B200_PLUGIN_COMMON_H
#define TENNIS_B200_PLUGIN_COMMON_H

#include <core/device_context.h>
#include <kernels/gpu/cuda_context.h>
#include <utils/ctxmgr_lite.h>
#include <utils/log.h>

#include "tennis_b200.h"

namespace ts {
    namespace b200 {
        // The workbench's own stream: every kernel of an operator is enqueued there and nobody synchronises
        // before a device-to-host view (what src/kernels/gpu/gpu_helper.cpp:98-106 does inside libtennis).
        inline cudaStream_t stream_on_context() {
            auto &context = ctx::ref<DeviceContext>();
            auto *handle = reinterpret_cast<CUDAContextHandle *>(context.handle);
            if (handle == nullptr) TS_LOG_ERROR << "The CUDAContextHandle is null! " << eject;
            return handle->stream();
        }

        // C-ABI status -> the exception TenniS operators raise
        inline void check(int status, const std::string &op) {
            if (status != TSB_OK) TS_LOG_ERROR << op << ": " << tsb_last_error() << " (status " << status << ")" << eject;
        }
    }
}

#endif
