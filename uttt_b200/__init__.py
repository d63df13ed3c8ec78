"""uttt_b200: a Blackwell-native universal test-time-training framework."""
__version__ = "0.1.0"
