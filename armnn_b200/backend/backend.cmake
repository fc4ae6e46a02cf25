# Build glue for dropping this directory into the Arm NN tree as src/backends/b200/ (src/backends/backends.cmake
# includes every backend.cmake it finds; the pattern is src/backends/reference/backend.cmake).
#
#   cmake -DARMNNB200=1 -DB200K_ROOT=/path/to/this/repository ...
#
# B200K_ROOT must hold include/b200k.h and a built armnn_b200/libb200k.so (python -m armnn_b200.build).

add_subdirectory(${PROJECT_SOURCE_DIR}/src/backends/b200)

if(ARMNNB200)
    list(APPEND armnnLibraries armnnB200Backend)
    list(APPEND armnnLinkLibraries ${ARMNN_B200_LINK_LIBRARIES})
else()
    message(STATUS "B200Acc backend is disabled")
endif()
