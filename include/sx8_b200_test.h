/* sx8_b200_test.h -- hooks of libsx8b200.so for its own test suite.  Not part of the
 * library's contract: applications include sx8_b200.h only. */
#ifndef SX8_B200_TEST_H
#define SX8_B200_TEST_H

#ifdef __cplusplus
extern "C" {
#endif

/* Force the GEMV's launch shape -- tile-group width (nt = 2, 4 or 8 tiles of 16 columns),
 * cluster split-K (1..8) and persistent grid size -- so that tests can run one product through
 * several shapes and compare; 0 = automatic for that field, -1 = back to the default rule.
 * Process-wide. */
void sx8_gemv_tune(int nt, int split, int grid);

#ifdef __cplusplus
}
#endif
#endif /* SX8_B200_TEST_H */
