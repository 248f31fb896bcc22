from .gemma import GemmaTokenizer, TokenizerError

__all__ = ["GemmaTokenizer", "TokenizerError"]
