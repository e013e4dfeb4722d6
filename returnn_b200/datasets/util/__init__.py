"""Dataset helpers: vocabularies, feature extraction."""
