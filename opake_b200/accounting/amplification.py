"""Amplification primitives are algorithm-specific (packages/opake-accounting/src/opake/api/accounting/core/amplification/
__init__.py): Poisson-family amplification lives in ``opake_b200.dpsgd.accounting`` (``poisson``, ``parallel_poisson``,
``k_out_of_t``), matrix-factorisation amplification in ``opake_b200.dpftrl.accounting`` (``poisson``, ``b_min_sep``,
``balls_in_bins``). This namespace exists so that ``accounting.amplification`` resolves, and is empty on purpose."""
__all__: list[str] = []
