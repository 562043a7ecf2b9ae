// The AVX-512 VNNI tier of the x86 int8 kernels (cera/src/backend/simd.rs:7288-9140): the same source as the AVX2
// tier with the byte dot product issued as vpdpbusd.  Test infrastructure, like the rest of this directory.
#define CERA_TIER_VNNI 1
#include "cera_cpu_avx2.cpp"
