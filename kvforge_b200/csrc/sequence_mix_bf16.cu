// The kernels of sequence_mix.cuh for bfloat16 storage (a translation unit per storage type: they compile side by side).
#include "sequence_mix.cuh"

KVF_SEQMIX_API(bf16, bf16)
