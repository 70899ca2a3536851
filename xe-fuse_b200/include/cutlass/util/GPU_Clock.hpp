// GPU_Clock: device-side stopwatch for the harness timing loops (CUDA events on the default stream).
#pragma once
#include <cuda_runtime_api.h>

struct GPU_Clock {
  GPU_Clock() { cudaEventCreate(&start_); cudaEventCreate(&stop_); }
  ~GPU_Clock() { cudaEventDestroy(start_); cudaEventDestroy(stop_); }
  GPU_Clock(GPU_Clock const&) = delete;
  GPU_Clock& operator=(GPU_Clock const&) = delete;
  void start() { cudaEventRecord(start_, 0); }
  float milliseconds() {
    cudaEventRecord(stop_, 0);
    cudaEventSynchronize(stop_);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, start_, stop_);
    return ms;
  }
  float seconds() { return milliseconds() * 1e-3f; }
 private:
  cudaEvent_t start_{}, stop_{};
};
