from kolmogorov_moe_architecture_b200.training.muon_optimizer import CombinedOptimizer, HybridOptimizer, Muon, Muon8bit, get_muon_optimizer  # noqa: F401
