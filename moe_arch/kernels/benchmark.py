from kolmogorov_moe_architecture_b200.kernels.benchmark import benchmark, create_test_data, main, verify_correctness  # noqa: F401

if __name__ == "__main__":
    main()
