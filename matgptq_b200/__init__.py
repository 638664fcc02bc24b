"""B200-native bit-sliced mixed-precision linear layer (MatGPTQ's serving hot path).

Importing the package does not load the CUDA library; importing ``matgptq_b200.ops``
(or anything built on it) does, and raises if it has not been built.
"""
__version__ = "0.1.0"
