// Stand-in for <torch/extension.h>, used only when the reference kernel sources
// are compiled into the parity checker (oracle/_ref/libdeltacnn_ref.so).
// The reference's common header names torch::Tensor in one declaration that the
// kernel translation units never call; an incomplete type satisfies it, so the
// checker library needs no libtorch. This is test infrastructure, not product code.
#pragma once
#include <exception>
#include <cstdio>
namespace torch { class Tensor; }
