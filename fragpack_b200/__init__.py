"""B200-native FragPack hot path: compressed-KV decode attention, block encoder, prefill decompressor.

The subpackages keep the names of the reference project (``compression``,
``ops``, ``integrations``) so that code written against it can switch by
changing the top-level package name.  ``fragpack_b200.ops`` is hand-written
sm_100a CUDA behind a C-ABI shared library; there is no CPU fallback.
"""

__version__ = "0.1.0"
