"""``poot`` command line: ``generate`` (llama-cli compatible flags), ``caption`` and ``embed``."""
