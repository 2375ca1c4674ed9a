// Stand-in for Vitis HLS <hls_math.h>: the operators call libm through <cmath>.
#pragma once
#include <cmath>
