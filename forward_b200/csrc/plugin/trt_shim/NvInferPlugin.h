// See NvInfer.h in this directory: stand-in used only when TensorRT is not installed.
#pragma once
#include "NvInfer.h"
