"""Helper services around the engine: API-key management, response store, tokenizer / detokenizer workers."""
