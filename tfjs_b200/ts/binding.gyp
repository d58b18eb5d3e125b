{
  "targets": [{
    "target_name": "tfjs_cuda_binding",
    "sources": ["binding/tfjs_cuda_binding.cc"],
    "include_dirs": ["../../include"],
    "libraries": ["-L<(module_root_dir)/..", "-ltfjs_cuda", "-Wl,-rpath,<(module_root_dir)/.."],
    "cflags_cc": ["-std=c++17", "-O2"],
    "defines": ["NAPI_VERSION=8"]
  }]
}
