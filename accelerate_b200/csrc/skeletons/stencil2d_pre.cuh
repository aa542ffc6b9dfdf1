// Register-window variant of the rank-2 stencil skeleton: taps are elements of
// per-thread windows w<input>_l<leaf>[ST_HW][ST_W<input>].  The window holds the
// ST_H = 2*ry+1 rows around the current output row plus ST2_DEPTH rows that have
// been requested ahead of time; its rows rotate with the phase PH of the row loop.
#define ST_REG 1
#ifndef ST2_DEPTH
#define ST2_DEPTH 4
#endif
#define ST_HW (ST_H + ST2_DEPTH)
#define ST_TAP(a, i, d0, d1, d2) w##a##_l##i[(PH + (d1) + ST_RYMAX + ST_HW) % ST_HW][K + (d2) + ST_R##a##_2]
