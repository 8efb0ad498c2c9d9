// The kernels of sequence_mix.cuh for float storage (a translation unit per storage type: they compile side by side).
#include "sequence_mix.cuh"

KVF_SEQMIX_API(f32, float)
