"""Test-support library: CPU oracle, input cases, wire spec, output checks and launch helpers.

Shipped with the package so external users can validate a build; not a runtime API.
"""
