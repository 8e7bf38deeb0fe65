"""Test oracle (CPU).  Test infrastructure only: the shipped package never imports this."""
