"""CPU oracles for the mapped-operator path -- TEST INFRASTRUCTURE ONLY.

``oracle.port``  plain-C restatement of the reference arithmetic (sph_oracle.c).
``oracle.ref``   the reference's own CPU modules, compiled by build_ref.py.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
package; the product package must never do so.
"""
