"""B200-native training backend for gguf-trainer's hot path.

`libgguftrain_cuda.so` (csrc/, C ABI in include/gguftrain.h) holds the device code. The Python
modules here are the host side a TypeScript caller would otherwise provide: they mirror the
reference's op interface (`autograd`), its device backend class (`backend.CudaBackend`, standing in
for `WebGPUBackend`), the three architectures, the optimizers and the step loops.
"""
