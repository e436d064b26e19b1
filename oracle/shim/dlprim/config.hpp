// Build configuration for the CPU-context checker build of the reference:
// no OpenCL wrapper selection, no sqlite cache, no ONNX/Caffe importers.
#pragma once
