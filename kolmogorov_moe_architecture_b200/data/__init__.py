from .dolma_dataset import (DolmaMemoryMappedDataset, DolmaStreamingDataset, PackedDocumentDataset,
                            PinnedPrefetcher, ThreadedPrefetcher, SyntheticTokenDataset, document_attention_mask, PackedDocs, get_dataloaders,
                            write_token_file)
from .tokenizer import ByteTokenizer, TokenizerWrapper
