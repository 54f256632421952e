"""Drop-in package layout: ``coda.kernels.functional`` backed by the B200 kernels of ``coda_kernels_b200``.

Putting this repository on ``sys.path`` ahead of the reference makes
``from coda.kernels.functional import swiglu as swiglu_functional`` (the import
style of the reference's benchmarks, benchmarks/linear.py:2-5) resolve to the
sm_100a implementation with unchanged call sites.
"""
