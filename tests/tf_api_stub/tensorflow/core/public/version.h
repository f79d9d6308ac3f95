// Declarations-only stand-in for TensorFlow's version header (type-check of the shims in the CPU suite).
#pragma once
#define TF_MAJOR_VERSION 2
#define TF_MINOR_VERSION 15
#define TF_PATCH_VERSION 0
