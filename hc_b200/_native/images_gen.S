.section .rodata
.balign 16
hc_img_name_0: .asciz "copy2d"
.balign 16
hc_img_begin_0: .incbin "/root/repo/hc_b200/_native/copy2d.cubin"
hc_img_end_0:
.balign 16
hc_img_name_1: .asciz "map_elements"
.balign 16
hc_img_begin_1: .incbin "/root/repo/hc_b200/_native/map_elements.cubin"
hc_img_end_1:
.balign 16
hc_img_name_2: .asciz "row_program"
.balign 16
hc_img_begin_2: .incbin "/root/repo/hc_b200/_native/row_program.cubin"
hc_img_end_2:
.balign 16
hc_img_name_3: .asciz "softmax_rows"
.balign 16
hc_img_begin_3: .incbin "/root/repo/hc_b200/_native/softmax_rows.cubin"
hc_img_end_3:
.balign 16
hc_img_name_4: .asciz "reduce_rows"
.balign 16
hc_img_begin_4: .incbin "/root/repo/hc_b200/_native/reduce_rows.cubin"
hc_img_end_4:
.balign 16
hc_img_name_5: .asciz "reduce_all"
.balign 16
hc_img_begin_5: .incbin "/root/repo/hc_b200/_native/reduce_all.cubin"
hc_img_end_5:
.balign 16
hc_img_name_6: .asciz "pairwise_distance"
.balign 16
hc_img_begin_6: .incbin "/root/repo/hc_b200/_native/pairwise_distance.cubin"
hc_img_end_6:
.balign 16
hc_img_name_7: .asciz "mapped_gemm"
.balign 16
hc_img_begin_7: .incbin "/root/repo/hc_b200/_native/mapped_gemm.cubin"
hc_img_end_7:
.balign 16
hc_img_name_8: .asciz "gemm_tiled"
.balign 16
hc_img_begin_8: .incbin "/root/repo/hc_b200/_native/gemm_tiled.cubin"
hc_img_end_8:
.balign 16
hc_img_name_9: .asciz "gemm_bf16_umma"
.balign 16
hc_img_begin_9: .incbin "/root/repo/hc_b200/_native/gemm_bf16_umma.cubin"
hc_img_end_9:
.balign 16
hc_img_name_10: .asciz "dequant_w8"
.balign 16
hc_img_begin_10: .incbin "/root/repo/hc_b200/_native/dequant_w8.cubin"
hc_img_end_10:
.balign 16
hc_img_name_11: .asciz "selftest"
.balign 16
hc_img_begin_11: .incbin "/root/repo/hc_b200/_native/selftest.cubin"
hc_img_end_11:
.balign 16
.section .data.rel.ro,"aw"
.globl hc_b200_images
.balign 8
hc_b200_images:
  .quad hc_img_name_0
  .quad hc_img_begin_0
  .quad hc_img_end_0
  .quad hc_img_name_1
  .quad hc_img_begin_1
  .quad hc_img_end_1
  .quad hc_img_name_2
  .quad hc_img_begin_2
  .quad hc_img_end_2
  .quad hc_img_name_3
  .quad hc_img_begin_3
  .quad hc_img_end_3
  .quad hc_img_name_4
  .quad hc_img_begin_4
  .quad hc_img_end_4
  .quad hc_img_name_5
  .quad hc_img_begin_5
  .quad hc_img_end_5
  .quad hc_img_name_6
  .quad hc_img_begin_6
  .quad hc_img_end_6
  .quad hc_img_name_7
  .quad hc_img_begin_7
  .quad hc_img_end_7
  .quad hc_img_name_8
  .quad hc_img_begin_8
  .quad hc_img_end_8
  .quad hc_img_name_9
  .quad hc_img_begin_9
  .quad hc_img_end_9
  .quad hc_img_name_10
  .quad hc_img_begin_10
  .quad hc_img_end_10
  .quad hc_img_name_11
  .quad hc_img_begin_11
  .quad hc_img_end_11
.section .rodata
.globl hc_b200_image_count
.balign 4
hc_b200_image_count:
  .long 12
.section .note.GNU-stack,"",@progbits
