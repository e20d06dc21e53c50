"""B200-native RL post-training compute platform.

Public surface mirrors the reference platform's: ``ArcticRLClientConfig`` and
``create_arctic_rl_client`` (see :mod:`arctic_platform_b200.rl` and
:mod:`arctic_platform_b200.client`), with the training, sampling and log-prob
engines implemented on hand-written sm_100a kernels (``csrc/``).
"""
__version__ = "0.1.0"

WIRE_FORMAT_VERSION = "DSSST1"
