"""Sequence and state mixers. Every mixer takes ``d_model`` (and ``layer_idx``) and maps ``[B, L, d] -> [B, L, d]``
causally; ``state_size(sequence_length)`` reports the recurrent state in elements."""
