// Tile geometry of the stencil skeleton; included before the generated code,
// which declares the shared-memory tiles and reads taps through ST_IDX<a>.
// Arrays of rank < 3 are padded with leading dimensions of extent 1.
// ST_T0..ST_T2: output tile extents (outermost first); ST_R<a>_<d>: halo radii.
#define ST_REG 0
#define ST_TAP(a, i, d0, d1, d2) sm##a##_l##i[ST_IDX##a(l0 + (d0), l1 + (d1), l2 + (d2))]
#define ST_P0_0 (ST_T0 + 2 * ST_R0_0)
#define ST_P0_1 (ST_T1 + 2 * ST_R0_1)
#define ST_P0_2 (ST_T2 + 2 * ST_R0_2)
#define ST_TILE_ELEMS0 (ST_P0_0 * ST_P0_1 * ST_P0_2)
#define ST_IDX0(z, y, x) ((((z) + ST_R0_0) * ST_P0_1 + ((y) + ST_R0_1)) * ST_P0_2 + ((x) + ST_R0_2))
#if ST_NIN > 1
#define ST_P1_0 (ST_T0 + 2 * ST_R1_0)
#define ST_P1_1 (ST_T1 + 2 * ST_R1_1)
#define ST_P1_2 (ST_T2 + 2 * ST_R1_2)
#define ST_TILE_ELEMS1 (ST_P1_0 * ST_P1_1 * ST_P1_2)
#define ST_IDX1(z, y, x) ((((z) + ST_R1_0) * ST_P1_1 + ((y) + ST_R1_1)) * ST_P1_2 + ((x) + ST_R1_2))
#endif
