// Empty build-configuration header for compiling the reference's quantized-decode
// headers against the host stand-in: no vendor library (cuBLAS, cuDNN, hipBLAS,
// MIOpen, Accelerate) is enabled, which is also what the quantized ops assume.
#pragma once
