"""CPU checker for the paged KV write/gather path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only ``tests/``, the smoke check and the CPU-baseline leg of ``bench.py`` import this
package.  ``kvx_b200`` never does.
"""
