"""CPU oracle for the grouped n:m path.  Test infrastructure only: the shipped package never imports it."""
