# CMake package of the bshmem runtime for C / C++ / CUDA consumers:
#
#   find_package(bshmem REQUIRED PATHS "$(bshmem-config --cmakedir)")
#   target_link_libraries(app PRIVATE bshmem::host)            # CPU backend, allocator, teams, proxy ring
#   target_link_libraries(gpu_app PRIVATE bshmem::cuda)        # NVLink backend + host API (needs the CUDA runtime)
#
# Device code includes <bshmem_device.cuh> / <bshmem_coll.cuh> (header-only; compile for sm_100a).
# Counterpart of the reference's exported roc_shmem target (library/CMakeLists.txt:90-295).
get_filename_component(_bshmem_pkg "${CMAKE_CURRENT_LIST_DIR}/.." ABSOLUTE)
set(bshmem_INCLUDE_DIR "${_bshmem_pkg}/csrc/include")
set(bshmem_LIBRARY_DIR "${_bshmem_pkg}/lib")
if(NOT EXISTS "${bshmem_LIBRARY_DIR}/libbshmem_host.so")
  message(FATAL_ERROR "bshmem: native libraries are not built; run `python -m roc_shmem_b200.build`")
endif()
if(NOT TARGET bshmem::host)
  add_library(bshmem::host SHARED IMPORTED)
  set_target_properties(bshmem::host PROPERTIES
    IMPORTED_LOCATION "${bshmem_LIBRARY_DIR}/libbshmem_host.so"
    INTERFACE_INCLUDE_DIRECTORIES "${bshmem_INCLUDE_DIR}")
endif()
if(EXISTS "${bshmem_LIBRARY_DIR}/libbshmem_cuda.so" AND NOT TARGET bshmem::cuda)
  add_library(bshmem::cuda SHARED IMPORTED)
  set_target_properties(bshmem::cuda PROPERTIES
    IMPORTED_LOCATION "${bshmem_LIBRARY_DIR}/libbshmem_cuda.so"
    INTERFACE_INCLUDE_DIRECTORIES "${bshmem_INCLUDE_DIR}")
endif()
set(bshmem_FOUND TRUE)
