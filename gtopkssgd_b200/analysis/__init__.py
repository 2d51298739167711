"""Offline analysis: communication cost models, the WFBP / merged-gradient
timeline simulator, log parsers and (optional, headless) figures."""
