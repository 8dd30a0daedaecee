"""Shape tables of the hot-path operators (counterpart of flextensor/configs/*.py)."""
