from kolmogorov_moe_architecture_b200.kernels.setup import get_cuda_arch_flags, get_cuda_version, get_gpu_arch, main  # noqa: F401

if __name__ == "__main__":
    main()
