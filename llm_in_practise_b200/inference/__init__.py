"""Generation: KV-cache runner, sampling, streaming, chat."""
from .generate import GenerationConfig, Generator, KVCache, TextIteratorStreamer, chat, sample_next, stream_generate
from .ragged import RaggedGenerator


def make_generator(model, tokenizer=None, max_len: int = 4096):
    """The runner that fits the model: ``RaggedGenerator`` for designs served by one ragged step, else ``Generator``."""
    base = getattr(model, "base_model", model)
    return (RaggedGenerator if getattr(base, "ragged", False) else Generator)(model, tokenizer, max_len)
