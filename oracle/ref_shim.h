// TEST INFRASTRUCTURE — compatibility shim for compiling the reference's own
// source/k3_moe_prefill_v4.cu with CUDA 12.9: that file uses the CUDA-13 vector type
// ulonglong4_16a (32 bytes, 16-byte aligned), which this toolkit does not define yet.
#pragma once
struct __align__(16) ulonglong4_16a { unsigned long long x, y, z, w; };
