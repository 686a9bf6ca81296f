from kolmogorov_moe_architecture_b200.data.dolma_dataset import DolmaMemoryMappedDataset, DolmaStreamingDataset, get_dataloaders  # noqa: F401
