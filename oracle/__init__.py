"""CPU oracle: test infrastructure for parity checks and the CPU baseline.

Nothing in the shipped package imports this.  `crypto` wraps the C
restatement (oracle/crypto_oracle.c) through ctypes, `crypto_py` is an
independent pure-Python restatement used to pin the C one, and `dl` restates
the five deep-learning operators with NumPy / PyTorch CPU ops.
"""
