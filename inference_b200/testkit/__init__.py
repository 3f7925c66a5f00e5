"""Conformance suites a third party can run against any provider, plus tiny synthetic snapshots for tests."""
