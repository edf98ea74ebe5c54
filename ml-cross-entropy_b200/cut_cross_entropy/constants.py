"""Constants shared by the host layer (reference: cut_cross_entropy/constants.py:2)."""

IGNORE_INDEX: int = -100
