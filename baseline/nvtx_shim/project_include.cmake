# Supplies the CUDA::nvToolsExt target that CUDA 12.9 no longer ships: header-only NVTX v3.
if(NOT TARGET CUDA::nvToolsExt)
  add_library(CUDA::nvToolsExt INTERFACE IMPORTED)
  target_include_directories(CUDA::nvToolsExt INTERFACE "${CMAKE_CURRENT_LIST_DIR}")
  target_link_libraries(CUDA::nvToolsExt INTERFACE ${CMAKE_DL_LIBS})
endif()
