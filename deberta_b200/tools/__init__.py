"""Developer tools shipped with the package.

* ``python -m deberta_b200.tools.audit_contracts``   — contract audit of the source tree (static + small dynamic checks)
* ``python -m deberta_b200.tools.kernel_drift_probe`` — PyTorch reference path vs CUDA kernel path, step by step
* ``python -m deberta_b200.tools.generate_api_docs``  — docstrings → ``docs/api/*.md``

They correspond to ``tools/audit_contracts.py``, ``tools/compile_drift_probe.py`` and ``tools/generate_api_docs.py``
of the reference; the drift probe compares the two execution paths this framework has (eager PyTorch oracle and
sm_100a kernels) instead of eager vs ``torch.compile``.
"""
