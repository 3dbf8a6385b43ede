"""CPU oracle of the reference's algorithms: test infrastructure only."""
