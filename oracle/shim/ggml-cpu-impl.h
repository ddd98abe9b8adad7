/* Test infrastructure only: empty stand-in for the fork's ggml-cpu-impl.h. */
#pragma once
