"""Input preparation of lookahead (multi-token) decoding steps for the paged cache (reference
``generation/parallel_decoding_mcore.py:19``)."""
import numpy as np


def la_pre_process(input_ids, slot_mapping, **model_kwargs):
    """A speculative step feeds every sequence ``q_seq_lens[b]`` tokens, padded per sequence to the longest. Returns the
    ``slot_mapping`` with the padding slots removed (one entry per real token, in sequence order) and the attention
    mask of the step (``spec_mask``, or a 1x1 zero when the step is plain)."""
    q_seq_lens = model_kwargs.get("q_seq_lens")
    if isinstance(q_seq_lens, int):          # warm-up passes a scalar: nothing to compact
        q_seq_lens = None
    if q_seq_lens is not None:
        q_seq_lens = [int(n) for n in q_seq_lens]
        total, widest = sum(q_seq_lens), max(q_seq_lens)
        slot_mapping = np.asarray(slot_mapping).reshape(-1)
        if slot_mapping.shape[0] != total:
            keep = np.concatenate([np.arange(b * widest, b * widest + n) for b, n in enumerate(q_seq_lens)])
            slot_mapping = slot_mapping[keep].astype(np.int32)
    mask = model_kwargs.get("spec_mask")
    if mask is None:
        mask = np.zeros((1, 1), dtype=np.float16)
    return slot_mapping, mask


def compact_padded_tokens(input_ids, q_seq_lens):
    """The tokens of a per-sequence padded ``[B, max(q_seq_lens)]`` step as one flat array of ``sum(q_seq_lens)``."""
    ids = np.asarray(input_ids).reshape(-1)
    q_seq_lens = [int(n) for n in q_seq_lens]
    widest = max(q_seq_lens)
    if ids.shape[0] == sum(q_seq_lens):
        return ids.astype(np.int32)
    keep = np.concatenate([np.arange(b * widest, b * widest + n) for b, n in enumerate(q_seq_lens)])
    return ids[keep].astype(np.int32)
