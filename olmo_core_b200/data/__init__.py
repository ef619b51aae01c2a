"""Data layer: collator, tokenizer configs, numpy datasets, data loaders and the composable source API."""
