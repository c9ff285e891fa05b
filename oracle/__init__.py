"""CPU oracle (test infrastructure): restatement of the reference's paged path."""
