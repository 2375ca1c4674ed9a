// Umbrella header: #include <flexllm/flexllm.hpp>
#pragma once
#include "FHT.hpp"
#include "HMT.hpp"
#include "LayerNorm.hpp"
#include "Linear_Layer.hpp"
#include "Logits.hpp"
#include "MHA.hpp"
#include "Residual_Layer.hpp"
#include "RoPE.hpp"
#include "Softmax.hpp"
#include "SpinQuant.hpp"
#include "Swish.hpp"
#include "quant.hpp"
