// Internal helpers of the host library.
#pragma once
#include <dlp_cuda.h>
#include <dlprim/definitions.hpp>

namespace dlprim {
namespace host {
    /// Throw DeviceError when a CUDA runtime call failed.
    void cuda_check(int err, char const *what);
    /// Map a C-ABI status to the reference's exception classes.
    void status_check(int status);
}
}
