// The activations an epilogue of a linear kernel can apply, in ONE list.  Every linear kernel includes this
// file: the code numbers, the functions and the dispatch from a run-time code to a compile-time one all come
// from the list below, and the Python side (parts/linear.py) reads the names and codes from this same file,
// so that a new activation is one more line here, its function in `activate`, and nothing else.
//
//   X(identifier, code, name)   name: how a configuration or a part spells it
#pragma once

#include <type_traits>

#include "common.cuh"

#define MLXB_ACTIVATION_LIST(X) \
  X(NONE, 0, none)              \
  X(GELU_NEW, 1, gelu_new)      \
  X(RELU, 2, relu)

#define MLXB_EPI_ENUM(ID, CODE, NAME) EPI_##ID = CODE,
enum { MLXB_ACTIVATION_LIST(MLXB_EPI_ENUM) };
#undef MLXB_EPI_ENUM
#define MLXB_EPI_COUNT_ONE(ID, CODE, NAME) +1
constexpr int EPI_COUNT = 0 MLXB_ACTIVATION_LIST(MLXB_EPI_COUNT_ONE);
#undef MLXB_EPI_COUNT_ONE

// The activation with code EPI on a float32 value.  FAST: the bfloat16 kernels' forms, built on the hardware
// exponential (errors far below bfloat16 resolution); otherwise the float32 path's forms with libm accuracy.
template <int EPI, bool FAST>
__device__ __forceinline__ float activate(float v) {
  if (EPI == EPI_GELU_NEW) return FAST ? gelu_new_fast(v) : gelu_new_f(v);
  if (EPI == EPI_RELU) return fmaxf(v, 0.f);
  return v;
}

// Calls fn(std::integral_constant<int, code>) for the run-time code `epi`; -1 if the code is not in the list.
template <typename Fn>
static inline int dispatch_activation(int epi, Fn&& fn) {
  switch (epi) {
#define MLXB_EPI_CASE(ID, CODE, NAME) \
  case CODE:                          \
    return fn(std::integral_constant<int, CODE>{});
    MLXB_ACTIVATION_LIST(MLXB_EPI_CASE)
#undef MLXB_EPI_CASE
  }
  return mlxb_fail(MLXB_BAD_ARG, "linear: epilogue code %d is not in the list of activations", epi);
}

static inline bool activation_known(int epi) { return epi >= 0 && epi < EPI_COUNT; }
