// Shared by the external-kernel fixtures: one output slot per SPMD block, a cache line apart.
#pragma once
constexpr int FLOATS_PER_CACHE_LINE = 16;
