from .dataset import Batch, Dataset, allocate_batches, collate, pack_sequences  # noqa: F401
