// Optional side interface of a GPU competitor: the device time of its last run_* in milliseconds, measured by the
// competitor itself with CUDA events on the stream(s) its kernels ran on.  The harness asks for it through a
// dynamic_cast to THIS interface (it never names a concrete competitor); a competitor without it is timed with the
// harness' own clock, as the reference does (src/benchmark/benchmark.hpp:159-168).
#pragma once

namespace SDDMM {

class DeviceTimed {
public:
    virtual float last_kernel_ms() = 0;

protected:
    ~DeviceTimed() = default;
};

}  // namespace SDDMM
