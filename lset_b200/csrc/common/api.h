// Launchers that other translation units of the library call.
#pragma once

extern "C" int lb_colsum(const float* partial, int P, int C, void* out, int out_fp32, int accumulate,
                         void* stream);
