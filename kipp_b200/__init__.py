"""kipp_b200: a small, whole inference engine for one GPU (NVIDIA B200,
sm_100a), for the Qwen3 dense decoder: configuration, weights, layers made of
parts, a paged cache, one step function, a scheduler, sampling, and the
hand-written CUDA kernels they run on."""

__version__ = "0.1.0"
