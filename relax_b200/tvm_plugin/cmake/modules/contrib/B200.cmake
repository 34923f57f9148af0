# B200 q4f16 kernel library: BYOC codegen + packed-function registration.
# Mirrors cmake/modules/contrib/CUTLASS.cmake:18-23 (codegen source into COMPILER_SRCS) and the
# USE_CURAND / USE_THRUST blocks of cmake/modules/CUDA.cmake (runtime sources + library link).
#   cmake -DUSE_CUDA=ON -DUSE_B200=/path/to/this/repo ..
if(USE_CUDA AND USE_B200)
  message(STATUS "Build with the B200 q4f16 kernel library from ${USE_B200}")
  include_directories(SYSTEM ${USE_B200}/include)
  tvm_file_glob(GLOB B200_CODEGEN_SRCS src/relax/backend/contrib/b200/*.cc)
  list(APPEND COMPILER_SRCS ${B200_CODEGEN_SRCS})
  tvm_file_glob(GLOB B200_RUNTIME_SRCS src/runtime/contrib/b200/*.cc)
  list(APPEND RUNTIME_SRCS ${B200_RUNTIME_SRCS})
  # the kernels themselves are prebuilt for sm_100a (python -m relax_b200.build)
  list(APPEND TVM_RUNTIME_LINKER_LIBS ${USE_B200}/relax_b200/libb200_q4f16.so)
endif()
