// Forwarding header: the generator implementation header moved to ATen/cuda/ in current PyTorch.
// Lets the unmodified reference sources compile against the installed torch.
#pragma once
#include <ATen/cuda/CUDAGeneratorImpl.h>
