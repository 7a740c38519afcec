"""CPU oracle of the HSA / HKV hot path.  Test infrastructure only: the product package never imports it."""
