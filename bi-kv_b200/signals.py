"""Task-type and hit/miss constants of the control plane.

Values follow ``DistributedStorage/Signals.py:4-12`` (the ``Signal`` enum inside
``protos/TaskInfo.proto:5-13`` carries different numbers and is unused by the
reference's code).
"""
SIGNAL_SEND = 1
SIGNAL_RECV = 2
SIGNAL_ACK = 3
SIGNAL_CHECK = 4
SIGNAL_SKIP = 5
SIGNAL_TERMINATE = -1

CACHE_MISS = 0
CACHE_HIT = 1
