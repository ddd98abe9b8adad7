/* Test infrastructure only: empty stand-in for the fork's ggml-backend.h. */
#pragma once
