"""B200-native training framework with the capabilities of the ml-experiments monorepo.

Sub-packages: ``ops`` (sm_100a kernels and their autograd wrappers), ``models``, ``optim``, ``parallel``,
``utils``, plus ``heuristic_secrets`` (byte-level secret detection pipeline) and ``zoology`` (synthetic-task
harness).
"""
__version__ = "0.1.0"
