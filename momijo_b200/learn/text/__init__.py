from .vocab import Vocab, build_vocab_from_iterator  # noqa: F401
