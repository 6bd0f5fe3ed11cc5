// The chunked (tensor-core) Gated DeltaNet kernel and its launcher (one translation unit of its own).
#define RQ_DN_CHUNK_INSTANTIATE
#include "deltanet_chunk.cuh"
