// Forwarding header: THC atomics now live in ATen/cuda/Atomic.cuh.
#pragma once
#include <ATen/cuda/Atomic.cuh>
