"""Measurement harness around the C ABI of ``libnvk.so``: seeded synthetic workloads, the single-kernel
benchmarks, and the torch decoder used to report end-to-end tokens per second.  Nothing here is part of the
product (``nano-vllm-cpp_b200/``: the C-ABI loader, ``csrc/`` and ``host/``); ``bench.py`` and the tests import it.
"""
