"""``python -m oneflow --doctor``: where the package lives, its version and how it was built
(reference: python/oneflow/__main__.py)."""
import argparse


def main(argv=None):
    parser = argparse.ArgumentParser(prog="python -m oneflow")
    parser.add_argument("--doctor", default=False, action="store_true", required=False)
    args = parser.parse_args(argv)
    if args.doctor:
        import torch

        import oneflow_b200 as flow
        from oneflow_b200 import sysconfig
        from oneflow_b200.ops import _native

        print("path:", list(flow.__path__))
        print("version:", flow.__version__)
        print("git_commit:", getattr(flow, "__git_commit__", "unknown"))
        print("cmake_build_type:", sysconfig.cmake_build_type())
        print("rdma:", sysconfig.with_rdma())
        print("mlir:", sysconfig.with_mlir())
        print("cuda:", sysconfig.with_cuda(), sysconfig.get_cuda_version())
        print("tensor substrate: torch", torch.__version__)
        print("native kernel library (sm_100a):", _native.lib_path("libofb_kernels.so"), "built" if _native.kernels_available() else "MISSING")
        print("native runtime library:", _native.lib_path("libofb_core.so"), "built" if _native.core_available() else "MISSING")
        import os
        api = _native.lib_path("libofb_api.so")
        print("graph compiler / C++ API library:", api, "built" if os.path.exists(api) else "MISSING")
        print("gpus:", torch.cuda.device_count(), [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())])
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
