"""Multi-head latent attention with DeepSeek sparse attention: cache rows, indexer, selection, absorbed attention."""
