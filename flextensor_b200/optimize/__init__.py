"""Command-line drivers: search, log and replay schedules per operator
(counterpart of flextensor/optimize/)."""
