// Stand-in for Vitis HLS <ap_fixed.h>: the operator path uses no fixed-point types.
#pragma once
