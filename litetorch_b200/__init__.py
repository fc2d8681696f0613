"""litetorch_b200: a Blackwell-native (sm_100a) LLM training engine with the LiteTorch API surface."""
__version__ = "0.1.0"
